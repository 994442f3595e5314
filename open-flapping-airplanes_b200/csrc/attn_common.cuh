// Shared definitions of the attention tasks (bf16 activations, head dim 64): tile sizes, the exp2-domain scale factors, and the
// row-term task of the backward pass.
//
// Layouts: qkv [N, 3D] (q | k | v, head h at columns h*64), o [N, D], lse/Dr [B, H, T] fp32, dqkv [N, 3D] (dq | dk | dv).
// A task covers 128 rows of one (sequence, head) pair and walks its partner rows 64 at a time (the reference's tiles cover 64
// rows, llm/attention/attention.cuh:81-516; its numerics - fp32 scores scaled by 0.125 * log2(e), running row maximum, P and dS
// rounded to bf16 before the products, lse in natural log - are kept by the tensor-core tasks in attn_tc.cuh).
#pragma once
#include "common.cuh"

namespace ofa {
namespace attn {

constexpr int DH = 64;
constexpr int QTILE = 128;      // rows per task
constexpr int KTILE = 64;       // partner rows per pipeline step
constexpr float SCALE = 0.125f;                       // 1/sqrt(64)
constexpr float SCALE_LOG2 = 0.125f * 1.4426950408889634f;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

// Dr[b,h,t] = sum_d dO[n, h*64+d] * O[n, h*64+d] (the reference's attn_bwd_prep_tile, attention.cuh:229-248). Task (b, h, rt)
// covers 128 rows; two threads per row. The training graph forms this term in the epilogue of the GEMM that produces dO instead
// (GE_DR); the task remains for callers at the task level that bring their own dO.
__device__ __forceinline__ void bwd_prep_task(const bf16* o, const bf16* dO, float* Dr, int b, int h, int rt, int T, int H) {
  const int D = H * DH;
  const int r = rt * QTILE + (threadIdx.x >> 1), half = threadIdx.x & 1;
  const size_t off = (size_t)(b * T + r) * D + h * DH + half * 32;
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < 4; c++) {
    float a[8], d[8];
    ldv(o + off + c * 8, a); ldv(dO + off + c * 8, d);
#pragma unroll
    for (int k = 0; k < 8; k++) s += a[k] * d[k];
  }
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  if (half == 0) Dr[((size_t)b * H + h) * T + r] = s;
}

}  // namespace attn
}  // namespace ofa
