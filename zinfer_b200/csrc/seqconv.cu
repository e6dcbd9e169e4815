// Causal depthwise convolution over time on the rows a mixer reads, with a residual term:
//   h_t = x_t + sum_{j < K} w[j, :] * x_{t - (K-1) + j}        (per channel; x before a sequence's start is 0)
// x is the float32 residual stream; the K-1 inputs before a step's first token come from the
// sequence's state [slots, K-1, D] (float32, row K-2 the most recent), which a second kernel
// moves on to the step's last K-1 inputs.  All arithmetic is float32 and the taps are added in
// the order of j, so a token's result does not depend on how its sequence was cut into steps.
// h is written in the run dtype (it is the input of the mixer's projections).
#include "common.cuh"
#include <stdint.h>

#define SEQCONV_MAX_TAPS 16

template <typename TO>
__global__ void seqconv_forward_kernel(const float* __restrict__ x, const float* __restrict__ state,
                                       const float* __restrict__ w, const int* __restrict__ tok_seq,
                                       const int* __restrict__ cu_q, const int* __restrict__ seq_slot,
                                       TO* __restrict__ h, int D, int K, long long state_stride, int residual) {
  zk_let_next_start();
  zk_wait_prior();
  const int t = blockIdx.x;
  const int b = tok_seq[t];
  const int o = t - cu_q[b];                     // offset of the token inside its sequence's part of the step
  const float* st = state + (size_t)seq_slot[b] * state_stride;
  for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < D; d += gridDim.y * blockDim.x) {
    const float cur = x[(size_t)t * D + d];
    float acc = 0.f;
    for (int j = 0; j < K; ++j) {
      const int src = o - (K - 1) + j;
      const float v = src >= 0 ? x[(size_t)(t - o + src) * D + d] : st[(size_t)(K - 1 + src) * D + d];
      acc = fmaf(w[(size_t)j * D + d], v, acc);
    }
    h[(size_t)t * D + d] = from_f32<TO>(residual ? cur + acc : acc);
  }
}

// The same four channels at a time (D a multiple of 4, 16-byte aligned rows): every value moves in 16-byte
// loads and the output in one store of four.  The sums are the scalar kernel's, term by term.
template <typename TO>
__global__ void seqconv_forward_vec4_kernel(const float* __restrict__ x, const float* __restrict__ state,
                                            const float* __restrict__ w, const int* __restrict__ tok_seq,
                                            const int* __restrict__ cu_q, const int* __restrict__ seq_slot,
                                            TO* __restrict__ h, int D, int K, long long state_stride, int residual) {
  zk_let_next_start();
  zk_wait_prior();
  const int t = blockIdx.x;
  const int b = tok_seq[t];
  const int o = t - cu_q[b];
  const float* st = state + (size_t)seq_slot[b] * state_stride;
  const int D4 = D >> 2;
  for (int d4 = blockIdx.y * blockDim.x + threadIdx.x; d4 < D4; d4 += gridDim.y * blockDim.x) {
    const float4 cur = reinterpret_cast<const float4*>(x + (size_t)t * D)[d4];
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < K; ++j) {
      const int src = o - (K - 1) + j;
      const float4 v = src >= 0 ? reinterpret_cast<const float4*>(x + (size_t)(t - o + src) * D)[d4]
                                : reinterpret_cast<const float4*>(st + (size_t)(K - 1 + src) * D)[d4];
      const float4 wv = reinterpret_cast<const float4*>(w + (size_t)j * D)[d4];
      acc.x = fmaf(wv.x, v.x, acc.x);
      acc.y = fmaf(wv.y, v.y, acc.y);
      acc.z = fmaf(wv.z, v.z, acc.z);
      acc.w = fmaf(wv.w, v.w, acc.w);
    }
    if (residual) {
      acc.x += cur.x;
      acc.y += cur.y;
      acc.z += cur.z;
      acc.w += cur.w;
    }
    if constexpr (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(h + (size_t)t * D)[d4] = acc;
    } else {
      __nv_bfloat162 pk[2] = {__floats2bfloat162_rn(acc.x, acc.y), __floats2bfloat162_rn(acc.z, acc.w)};
      reinterpret_cast<uint2*>(h + (size_t)t * D)[d4] = *reinterpret_cast<const uint2*>(pk);
    }
  }
}

// state[slot] <- the last K-1 inputs of the sequence (older rows move up if fewer tokens came).
// One thread per (sequence, channel) reads everything it needs before it writes.
__global__ void seqconv_state_update_kernel(const float* __restrict__ x, float* __restrict__ state,
                                            const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int D,
                                            int K, long long state_stride) {
  zk_let_next_start();
  zk_wait_prior();
  const int b = blockIdx.x;
  const int t0 = cu_q[b], L = cu_q[b + 1] - t0;
  float* st = state + (size_t)seq_slot[b] * state_stride;
  for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < D; d += gridDim.y * blockDim.x) {
    float keep[SEQCONV_MAX_TAPS - 1];
#pragma unroll
    for (int r = 0; r < SEQCONV_MAX_TAPS - 1; ++r) {
      if (r >= K - 1) break;
      const int src = L - (K - 1) + r;
      keep[r] = src >= 0 ? x[(size_t)(t0 + src) * D + d] : st[(size_t)(K - 1 + src) * D + d];
    }
#pragma unroll
    for (int r = 0; r < SEQCONV_MAX_TAPS - 1; ++r) {
      if (r >= K - 1) break;
      st[(size_t)r * D + d] = keep[r];
    }
  }
}

// One token per sequence (row b = sequence b): the convolution and the state's shift in one kernel.
template <typename TO>
__global__ void seqconv_single_kernel(const float* __restrict__ x, float* __restrict__ state,
                                      const float* __restrict__ w, const int* __restrict__ seq_slot,
                                      TO* __restrict__ h, int D, int K, long long state_stride, int residual) {
  zk_let_next_start();
  zk_wait_prior();
  const int b = blockIdx.x;
  float* st = state + (size_t)seq_slot[b] * state_stride;
  for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < D; d += gridDim.y * blockDim.x) {
    const float cur = x[(size_t)b * D + d];
    float acc = 0.f;
    for (int j = 0; j < K - 1; ++j) {
      const float v = st[(size_t)j * D + d];
      acc = fmaf(w[(size_t)j * D + d], v, acc);
      if (j > 0) st[(size_t)(j - 1) * D + d] = v;
    }
    acc = fmaf(w[(size_t)(K - 1) * D + d], cur, acc);
    if (K > 1) st[(size_t)(K - 2) * D + d] = cur;
    h[(size_t)b * D + d] = from_f32<TO>(residual ? cur + acc : acc);
  }
}

extern "C" {

int zk_seqconv_max_taps() { return SEQCONV_MAX_TAPS; }

// x [n, D] float32; state [slots, K-1, D] float32 (slot stride given); w [K, D] float32 (tap, channel);
// h [n, D] in `out_dtype`.  single != 0: one token per sequence, the state moves on in the same kernel;
// otherwise the state is only read and zk_seqconv_state_update follows.
int zk_seqconv_forward(const float* x, float* state, const float* w, const int* tok_seq, const int* cu_q,
                       const int* seq_slot, void* h, int n, int D, int K, long long state_stride, int residual,
                       int single, int out_dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (D <= 0 || K < 1 || K > SEQCONV_MAX_TAPS || (out_dtype != ZK_F32 && out_dtype != ZK_BF16)) return ZK_EINVAL;
  const int threads = D >= 256 ? 256 : (D >= 128 ? 128 : 64);
  const dim3 grid(n, ceil_div_i(D, threads));
  if (single) {
    if (out_dtype == ZK_F32)
      return zk_launch_dependent(seqconv_single_kernel<float>, grid, dim3(threads), 0, stream, x, state, w, seq_slot, (float*)h, D, K, state_stride, residual);
    return zk_launch_dependent(seqconv_single_kernel<bf16>, grid, dim3(threads), 0, stream, x, state, w, seq_slot, (bf16*)h, D, K, state_stride, residual);
  }
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(state) | reinterpret_cast<uintptr_t>(w) |
                         reinterpret_cast<uintptr_t>(h)) % 16) == 0;
  if (D % 4 == 0 && state_stride % 4 == 0 && aligned) {
    const int t4 = D >= 1024 ? 256 : (D >= 512 ? 128 : 64);
    const dim3 grid4(n, ceil_div_i(D / 4, t4));
    if (out_dtype == ZK_F32)
      return zk_launch_dependent(seqconv_forward_vec4_kernel<float>, grid4, dim3(t4), 0, stream, x, (const float*)state, w, tok_seq, cu_q, seq_slot, (float*)h, D, K, state_stride, residual);
    return zk_launch_dependent(seqconv_forward_vec4_kernel<bf16>, grid4, dim3(t4), 0, stream, x, (const float*)state, w, tok_seq, cu_q, seq_slot, (bf16*)h, D, K, state_stride, residual);
  }
  if (out_dtype == ZK_F32)
    return zk_launch_dependent(seqconv_forward_kernel<float>, grid, dim3(threads), 0, stream, x, (const float*)state, w, tok_seq, cu_q, seq_slot, (float*)h, D, K, state_stride, residual);
  return zk_launch_dependent(seqconv_forward_kernel<bf16>, grid, dim3(threads), 0, stream, x, (const float*)state, w, tok_seq, cu_q, seq_slot, (bf16*)h, D, K, state_stride, residual);
}

int zk_seqconv_state_update(const float* x, float* state, const int* cu_q, const int* seq_slot, int n_seqs, int D,
                            int K, long long state_stride, cudaStream_t stream) {
  if (n_seqs <= 0 || K <= 1) return 0;
  if (D <= 0 || K > SEQCONV_MAX_TAPS) return ZK_EINVAL;
  const int threads = D >= 256 ? 256 : (D >= 128 ? 128 : 64);
  return zk_launch_dependent(seqconv_state_update_kernel, dim3(n_seqs, ceil_div_i(D, threads)), dim3(threads), 0,
                             stream, x, state, cu_q, seq_slot, D, K, state_stride);
}

}  // extern "C"
