/* Pulls in the C ABI of the CUDA backend; pass -Xcc -I<repository>/include when building. */
#include "metalaudio_cuda.h"
