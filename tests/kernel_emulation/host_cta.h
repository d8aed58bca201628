// CPU emulation of a CUDA thread block for the test-suite: one OS thread per CUDA
// thread and a pthread barrier for __syncthreads().  TEST INFRASTRUCTURE ONLY: it
// lets the kernels' index arithmetic be executed and checked where no GPU exists; it is
// never linked into the product library.
#pragma once
#include <pthread.h>

#include <functional>
#include <thread>
#include <vector>

struct HostCta {
    int tid_, bid_, nblocks_;
    pthread_barrier_t* bar_;
    int tid() const { return tid_; }
    int bid() const { return bid_; }
    int nblocks() const { return nblocks_; }
    void sync() { pthread_barrier_wait(bar_); }
};

// Runs `body(cta, smem)` for every thread of every block of a 1-D grid, blocks one
// after another, the threads of a block concurrently.
inline void run_grid(int nblocks, int nthreads, size_t smem_bytes,
                     const std::function<void(HostCta&, void*)>& body) {
    for (int b = 0; b < nblocks; ++b) {
        std::vector<char> smem(smem_bytes + 64);
        pthread_barrier_t bar;
        pthread_barrier_init(&bar, nullptr, nthreads);
        std::vector<std::thread> th;
        th.reserve(nthreads);
        for (int t = 0; t < nthreads; ++t) {
            th.emplace_back([&, t]() {
                HostCta cta{t, b, nblocks, &bar};
                body(cta, smem.data());
            });
        }
        for (auto& x : th) x.join();
        pthread_barrier_destroy(&bar);
    }
}
