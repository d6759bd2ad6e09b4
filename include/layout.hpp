#pragma once
// Drop-in for the reference's src/runtime/layout.hpp (lines 5-9):
// [32, tokens, 64] -> [tokens, 2048] on the default stream; a launch error
// prints and exits as in src/runtime/layout.cu:64-75.
#include <cstdio>
#include <cstdlib>
#include <cuda_bf16.h>

// Defined in libpaged_attention.so (csrc/compat_cxx.cu) with this exact C++ signature.
void launch_flash_output_layout(const __nv_bfloat16* input, __nv_bfloat16* output, int tokens);
