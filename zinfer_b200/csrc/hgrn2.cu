// Gated linear recurrence with a matrix state per head (HGRN2): per head a state S [d, e],
//
//     S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T,        o_t = S_t^T q_t,
//
// f_t in (lower, 1) the forget gate per head and channel, which also decides how much of v_t is written
// (there is no key), q_t = silu(.), v_t plain.  A row of `qfv` holds the three projections of a token,
// [q (H*d) | f (H*d) | v (H*e)], float32 as the contraction left them; the gate is
// f = lower + (1 - lower) * sigmoid(z_f + bias).  Everything here is float32: gate, state, sums.
//
// One kernel serves prompt steps and single-token steps.  A block owns one (sequence, head, stretch of
// value columns); a thread owns one column of S (d values in registers) and walks the sequence's
// tokens in order, from the state the step before left in `state[slot]` to the state it leaves there.
// q, f and 1 - f of eight tokens at a time are staged in shared memory (activations applied once per
// block), every thread reads them as broadcasts.  The sum over a column runs over the channels in
// ascending order whatever the step's shape, so a sequence cut into steps gives the same bits.
#include "common.cuh"
#include <math.h>

#define HG_TT 8            // tokens staged at once
#define HG_MAX_D 256
#define HG_MAX_COLS 128    // value columns (threads) per block

template <int DMAX>
__global__ void __launch_bounds__(HG_MAX_COLS)
    hgrn2_scan_kernel(const float* __restrict__ qfv, int ld, const float* __restrict__ f_bias,
                      const float* __restrict__ lower, float* __restrict__ state, long long state_stride,
                      float* __restrict__ o, const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int H, int d,
                      int e) {
  __shared__ __align__(16) float qs[HG_TT][DMAX];
  __shared__ __align__(16) float fs[HG_TT][DMAX];
  __shared__ __align__(16) float gs[HG_TT][DMAX];
  const int b = blockIdx.x, h = blockIdx.y;
  const int c = blockIdx.z * blockDim.x + threadIdx.x;
  const bool col = c < e;
  zk_let_next_start();
  zk_wait_prior();   // qfv is the kernel before's result
  const int t0 = cu_q[b], t1 = cu_q[b + 1];
  float* st = state + (size_t)seq_slot[b] * state_stride + (size_t)h * d * e;
  float S[DMAX];
#pragma unroll
  for (int i = 0; i < DMAX; ++i) S[i] = (col && i < d) ? st[(size_t)i * e + c] : 0.f;

  const int off_f = H * d, off_v = 2 * H * d;
  for (int tb = t0; tb < t1; tb += HG_TT) {
    const int nt = min(HG_TT, t1 - tb);
    __syncthreads();   // the tokens staged before are consumed
    for (int idx = threadIdx.x; idx < nt * d; idx += blockDim.x) {
      const int tt = idx / d, i = idx - tt * d;
      const float* row = qfv + (size_t)(tb + tt) * ld;
      const float zq = row[h * d + i];
      const float zf = row[off_f + h * d + i] + f_bias[h * d + i];
      const float lo = lower[h * d + i];
      const float f = lo + (1.0f - lo) * (1.0f / (1.0f + expf(-zf)));
      qs[tt][i] = zq / (1.0f + expf(-zq));
      fs[tt][i] = f;
      gs[tt][i] = 1.0f - f;
    }
    float v[HG_TT];
#pragma unroll
    for (int tt = 0; tt < HG_TT; ++tt)
      v[tt] = (col && tt < nt) ? qfv[(size_t)(tb + tt) * ld + off_v + h * e + c] : 0.f;
    __syncthreads();
#pragma unroll
    for (int tt = 0; tt < HG_TT; ++tt) {
      if (tt >= nt) break;
      float acc = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < DMAX; i4 += 4) {
        if (i4 < d) {
          const float4 f4 = *reinterpret_cast<const float4*>(&fs[tt][i4]);
          const float4 g4 = *reinterpret_cast<const float4*>(&gs[tt][i4]);
          const float4 q4 = *reinterpret_cast<const float4*>(&qs[tt][i4]);
          const float ff[4] = {f4.x, f4.y, f4.z, f4.w}, gg[4] = {g4.x, g4.y, g4.z, g4.w},
                      qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (i4 + j < d) {
              S[i4 + j] = fmaf(ff[j], S[i4 + j], gg[j] * v[tt]);
              acc = fmaf(S[i4 + j], qq[j], acc);
            }
          }
        }
      }
      if (col) o[(size_t)(tb + tt) * H * e + (size_t)h * e + c] = acc;
    }
  }
  if (col) {
#pragma unroll
    for (int i = 0; i < DMAX; ++i)
      if (i < d) st[(size_t)i * e + c] = S[i];
  }
}

extern "C" {

int zk_hgrn2_max_dim() { return HG_MAX_D; }

// qfv float32 [n, >= 2*H*d + H*e] with rows `ld` floats apart; f_bias, lower float32 [H*d]; state float32, a
// slot's [H, d, e] block `state_stride` floats after the one before; o float32 [n, H*e]; cu_q [n_seqs + 1],
// seq_slot [n_seqs].
int zk_hgrn2_scan(const float* qfv, int ld, const float* f_bias, const float* lower, float* state, long long state_stride,
                  float* o, const int* cu_q, const int* seq_slot, int n_seqs, int H, int d, int e, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (H <= 0 || d <= 0 || e <= 0 || d > HG_MAX_D || ld < 2 * H * d + H * e || !f_bias || !lower) return ZK_EINVAL;
  int threads = 32;
  while (threads < HG_MAX_COLS && threads < e) threads <<= 1;
  dim3 grid(n_seqs, H, (e + threads - 1) / threads);
#define ZK_HG(DM)                                                                                                   \
  return zk_launch_dependent(hgrn2_scan_kernel<DM>, grid, dim3(threads), 0, stream, qfv, ld, f_bias, lower, state,  \
                             state_stride, o, cu_q, seq_slot, H, d, e)
  if (d <= 16) ZK_HG(16);
  if (d <= 32) ZK_HG(32);
  if (d <= 64) ZK_HG(64);
  if (d <= 128) ZK_HG(128);
  ZK_HG(256);
#undef ZK_HG
}

}  // extern "C"
