// CPU emulation of a CUDA thread block for the test-suite: one OS thread per CUDA
// thread and a pthread barrier for __syncthreads().  TEST INFRASTRUCTURE ONLY: it
// lets the kernels' index arithmetic be executed and checked where no GPU exists; it is
// never linked into the product library.
#pragma once
#include <pthread.h>
#include <sched.h>
#include <string.h>

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
    // Bulk asynchronous copy emulated as an immediate copy that then bumps a completion count
    // in the barrier word.  The producer is never more than one copy ahead of the waiters, so
    // the k-th wait (parity k & 1) is satisfied exactly when the count's low bit differs from it.
    void bulk_init(void* bar) { __atomic_store_n((unsigned long long*)bar, 0ull, __ATOMIC_SEQ_CST); }
    void bulk_copy(void* dst, const void* src, unsigned bytes, void* bar) {
        memcpy(dst, src, bytes);
        __atomic_add_fetch((unsigned long long*)bar, 1ull, __ATOMIC_SEQ_CST);
    }
    // Several copies on one phase: the parts are copied at once and the count is bumped when the
    // bytes announced by bulk_expect have all arrived (one thread issues them, in program order).
    unsigned pending_ = 0;
    void bulk_expect(void* bar, unsigned total_bytes) {
        (void)bar;
        pending_ = total_bytes;
    }
    void bulk_part(void* dst, const void* src, unsigned bytes, void* bar) {
        memcpy(dst, src, bytes);
        pending_ -= bytes;
        if (pending_ == 0) __atomic_add_fetch((unsigned long long*)bar, 1ull, __ATOMIC_SEQ_CST);
    }
    bool bulk_wait(void* bar, unsigned parity) {
        for (long i = 0; i < (1L << 21); ++i) {
            if ((__atomic_load_n((unsigned long long*)bar, __ATOMIC_SEQ_CST) & 1ull) == (unsigned long long)(parity ^ 1u))
                return true;
            sched_yield();
        }
        return false;
    }
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
