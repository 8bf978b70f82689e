// The quantized linear for many rows of activations (prefill-sized M) on the tensor cores:
// declarations shared by qlinear_tc.cu (the kernel) and qlinear.cu (the entry point).
#pragma once

#include <stdint.h>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace dgq {

struct QLinearTcArgs {
  const void* x; void* y;               // (M, K) and (M, N_out), row-major, dtype DGQ_F16 or DGQ_BF16
  int dtype;
  const uint8_t* qw; int64_t row_bytes; // (N_out, K/2): two 4-bit codes per byte, even column low
  const __half* scales; const __half* zeros; int n_groups, group_size;
  const void* bias; int bias_dtype;     // may be null
  int M, N_out, K;
  int32_t* info;                        // device status words for bounded-wait timeouts, may be null
};

// True when the kernel takes the problem: 16-bit activations, K a multiple of 64, groups of a
// multiple of 64 consecutive columns (or one group), 16-byte aligned rows of codes.
bool qlinear_tc_supported(const QLinearTcArgs& a);
// Enqueues the product on `st`; false if the tensor map could not be encoded or the launch failed.
bool qlinear_tc_launch(const QLinearTcArgs& a, cudaStream_t st);

}  // namespace dgq
