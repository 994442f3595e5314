// fp32 SIMT tasks for the tiny model (widths that are not multiples of the tensor-core tile: D=64, head dim 16, V=65).
// Same task contract, layouts and epilogues as the bf16 path; every sum has a fixed order (one thread owns one output and
// walks k upwards), so results are bitwise independent of the schedule. Speed is not a goal here.
#pragma once
#include "common.cuh"
#include "task_api.h"

namespace ofa {
namespace f32 {

constexpr int GT = 64;     // output tile edge
constexpr int GK = 16;     // k per shared-memory step
constexpr int GEMM_SMEM = 2 * GT * GK * 4;

template <int LAYOUT> __device__ __forceinline__ float ld_a(const GemmArgs& g, int m, int k) {
  const float* A = reinterpret_cast<const float*>(g.A);
  if (m >= g.M || k >= g.K) return 0.f;
  return LAYOUT == GL_TN ? A[(size_t)k * g.lda + m] : A[(size_t)m * g.lda + k];
}
template <int LAYOUT> __device__ __forceinline__ float ld_b(const GemmArgs& g, int k, int n) {
  const float* B = reinterpret_cast<const float*>(g.B);
  if (n >= g.N || k >= g.K) return 0.f;
  return LAYOUT == GL_NT ? B[(size_t)n * g.ldb + k] : B[(size_t)k * g.ldb + n];
}

// one 64x64 tile of C; task -> (tm = task % tiles_m, tn = task / tiles_m); thread (ty, tx) owns a 4x4 block
template <int LAYOUT>
__device__ __forceinline__ void gemm_task(const GemmArgs& g, int epi, int tiles_m, int task, unsigned char* smem) {
  float* sA = reinterpret_cast<float*>(smem);          // [GK][GT]  (k-major so the inner loop reads contiguous rows)
  float* sB = sA + GT * GK;                            // [GK][GT]
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int m0 = (task % tiles_m) * GT, n0 = (task / tiles_m) * GT;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
  for (int k0 = 0; k0 < g.K; k0 += GK) {
    for (int i = tid; i < GT * GK; i += NTHR) {
      const int kk = i / GT, mm = i % GT;
      sA[kk * GT + mm] = ld_a<LAYOUT>(g, m0 + mm, k0 + kk);
      sB[kk * GT + mm] = ld_b<LAYOUT>(g, k0 + kk, n0 + mm);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < GK; kk++) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; i++) { a[i] = sA[kk * GT + ty * 4 + i]; b[i] = sB[kk * GT + tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  float* C = reinterpret_cast<float*>(g.C);
  float* aux = reinterpret_cast<float*>(g.aux);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int m = m0 + ty * 4 + i;
    if (m >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int n = n0 + tx * 4 + j;
      if (n >= g.N) continue;
      float v = acc[i][j];
      const size_t ci = (size_t)m * g.ldc + n, ai = (size_t)m * g.ldaux + n;
      switch (epi) {
        case GE_RES: v += aux[ai]; break;
        case GE_GELU: aux[ai] = v; v = gelu_fwd<false>(v); break;
        case GE_DGELU: v *= gelu_bwd<false>(aux[ai]); break;
        case GE_F32: if (g.accumulate) v += C[ci]; break;
        default: break;
      }
      C[ci] = v;
    }
  }
  __syncthreads();
}
__device__ __noinline__ void gemm_run(const PhaseDesc& d, int task, unsigned char* smem) {
  switch (d.layout) {
    case GL_NN: gemm_task<GL_NN>(d.g, d.epi, d.tiles_m, task, smem); break;
    case GL_NT: gemm_task<GL_NT>(d.g, d.epi, d.tiles_m, task, smem); break;
    default:    gemm_task<GL_TN>(d.g, d.epi, d.tiles_m, task, smem); break;
  }
}

// ---------------------------------------------------------------------------------------------- attention (one task per (b, h))
__host__ __device__ constexpr size_t attn_fwd_smem(int T, int DH) { return (size_t)(3 * T * DH + T * T) * 4; }
__host__ __device__ constexpr size_t attn_bwd_smem(int T, int DH) { return (size_t)(5 * T * DH + 2 * T * T + T) * 4; }

template <int DH>
__device__ __forceinline__ void attn_fwd_task(const float* qkv, float* o, float* lse, int b, int h, int T, int H, unsigned char* smem) {
  const int D = H * DH, ld = 3 * D;
  float* sq = reinterpret_cast<float*>(smem); float* sk = sq + T * DH; float* sv = sk + T * DH; float* sp = sv + T * DH;
  const float scale = rsqrtf((float)DH);
  for (int i = threadIdx.x; i < T * DH; i += NTHR) {
    const int r = i / DH, c = i % DH;
    const float* row = qkv + (size_t)(b * T + r) * ld + h * DH + c;
    sq[i] = row[0]; sk[i] = row[D]; sv[i] = row[2 * D];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < T; i += NTHR) {
    float m = -INFINITY;
    for (int j = 0; j <= i; j++) {
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < DH; c++) s = fmaf(sq[i * DH + c], sk[j * DH + c], s);
      s *= scale; sp[i * T + j] = s; m = fmaxf(m, s);
    }
    float l = 0.f;
    for (int j = 0; j <= i; j++) { const float p = expf(sp[i * T + j] - m); sp[i * T + j] = p; l += p; }
    const float inv = 1.f / l;
#pragma unroll
    for (int c = 0; c < DH; c++) {
      float a = 0.f;
      for (int j = 0; j <= i; j++) a = fmaf(sp[i * T + j], sv[j * DH + c], a);
      o[(size_t)(b * T + i) * D + h * DH + c] = a * inv;
    }
    lse[((size_t)b * H + h) * T + i] = m + logf(l);
  }
  __syncthreads();
}

// dq | dk | dv for one (b, h): recomputes P from lse, D = rowsum(dO * O), dS = P * (dP - D).
template <int DH>
__device__ __forceinline__ void attn_bwd_task(const float* qkv, const float* o, const float* dO, const float* lse, float* dqkv,
                                              int b, int h, int T, int H, unsigned char* smem) {
  const int D = H * DH, ld = 3 * D;
  float* sq = reinterpret_cast<float*>(smem); float* sk = sq + T * DH; float* sv = sk + T * DH; float* sdo = sv + T * DH; float* so = sdo + T * DH;
  float* sp = so + T * DH; float* sds = sp + T * T; float* sD = sds + T * T;
  const float scale = rsqrtf((float)DH);
  for (int i = threadIdx.x; i < T * DH; i += NTHR) {
    const int r = i / DH, c = i % DH;
    const float* row = qkv + (size_t)(b * T + r) * ld + h * DH + c;
    sq[i] = row[0]; sk[i] = row[D]; sv[i] = row[2 * D];
    sdo[i] = dO[(size_t)(b * T + r) * D + h * DH + c]; so[i] = o[(size_t)(b * T + r) * D + h * DH + c];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < T; i += NTHR) {
    float d = 0.f;
#pragma unroll
    for (int c = 0; c < DH; c++) d = fmaf(sdo[i * DH + c], so[i * DH + c], d);
    sD[i] = d;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < T * T; e += NTHR) {
    const int i = e / T, j = e % T;
    float p = 0.f, ds = 0.f;
    if (j <= i) {
      float s = 0.f, dp = 0.f;
#pragma unroll
      for (int c = 0; c < DH; c++) { s = fmaf(sq[i * DH + c], sk[j * DH + c], s); dp = fmaf(sdo[i * DH + c], sv[j * DH + c], dp); }
      p = expf(s * scale - lse[((size_t)b * H + h) * T + i]);
      ds = p * (dp - sD[i]);
    }
    sp[e] = p; sds[e] = ds;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < T * DH; e += NTHR) {
    const int r = e / DH, c = e % DH;
    float dq = 0.f, dk = 0.f, dv = 0.f;
    for (int j = 0; j <= r; j++) dq = fmaf(sds[r * T + j], sk[j * DH + c], dq);
    for (int i = r; i < T; i++) { dk = fmaf(sds[i * T + r], sq[i * DH + c], dk); dv = fmaf(sp[i * T + r], sdo[i * DH + c], dv); }
    float* row = dqkv + (size_t)(b * T + r) * ld + h * DH + c;
    row[0] = dq * scale; row[D] = dk * scale; row[2 * D] = dv;
  }
  __syncthreads();
}

}  // namespace f32
}  // namespace ofa
