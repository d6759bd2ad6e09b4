#ifndef ROPE_HPP
#define ROPE_HPP
// Drop-in for the reference's src/kernels/rope/rope.hpp (lines 11-63): the
// same constants and the same launch_rope_qkv signature.  Like the reference's
// launcher (src/kernels/rope/rope.cu:305-358) it returns with the results
// complete: it runs on the default stream and synchronises the device.
#include <cstdio>
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

constexpr int ROPE_HEADS = 32;
constexpr int ROPE_KV_HEADS = 8;
constexpr int ROPE_HEAD_DIM = 64;
constexpr int ROPE_BLOCK_SIZE = 256;
constexpr int ROPE_ROTARY_DIM = ROPE_HEAD_DIM / 2;

#ifndef CUDA_CHECK
#define CUDA_CHECK(call)                                      \
do {                                                          \
    cudaError_t err = call;                                   \
    if(err != cudaSuccess)                                    \
    {                                                         \
        printf("CUDA Error %s:%d : %s\n", __FILE__, __LINE__, \
               cudaGetErrorString(err));                      \
        exit(EXIT_FAILURE);                                   \
    }                                                         \
} while(0)
#endif

// Defined in libpaged_attention.so (csrc/compat_cxx.cu) with this exact C++ signature.
void launch_rope_qkv(const __nv_bfloat16* q_in, __nv_bfloat16* q_out,
                     const __nv_bfloat16* k_in, __nv_bfloat16* k_out,
                     const __nv_bfloat16* v_in, __nv_bfloat16* v_out,
                     float* cos_table, float* sin_table, int tokens,
                     int position_offset);

#endif
