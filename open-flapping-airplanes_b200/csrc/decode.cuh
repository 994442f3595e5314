// Batch-1 KV-cache decode from the LIVE working-copy weights, as tasks of the serving job.
//
// Phase structure, task granularity and every rounding point follow the reference's decode task set
// (llm/b200/megakernel/decode_wide.cuh:251-626): per layer QKV (LN1 prologue + 64-column GEMV slice, K/V row appended at
// `pos`), ATT+WO (one head's softmax attention + its slice of Wo), UP+DOWN (LN2 + 64 hidden units + their slice of Wdown);
// then HEAD (LN_f + 128 vocabulary rows per task, fp32 logits, chunk-local argmax / Gumbel-max) and SAMPLE (fixed-order
// final pick, prompt forcing / answer mode, position update, next embedding). The residual stream is kept in int64 fixed
// point (2^-30 units) and updated with integer atomics, so the result is bitwise independent of task order. LN output,
// attention output and GELU output are each rounded to the activation type T before the next product; q, K, V are stored
// as T; softmax uses expf; GELU uses tanhf; argmax ties go to the lower index and NaN never wins.
// Weight and KV loads bypass L1 so that weights refreshed by AdamW on other SMs are seen; nothing synchronises the
// decoder with the trainer.
//
// Unlike the reference, the code is generic over T in {bf16, float}, the width D and the head dim DH (the thread mappings
// are derived from the 16-byte vector width), so the tiny fp32 model runs through the same tasks.
#pragma once
#include "common.cuh"
#include "task_api.h"

namespace ofa {
namespace dec {

constexpr int HR = 128;                               // vocabulary rows per head task
constexpr float FX_SCALE = 1073741824.0f;             // 2^30
constexpr float FX_INV = 1.0f / 1073741824.0f;
__device__ __forceinline__ unsigned long long fx(float v) { return (unsigned long long)llrintf(v * FX_SCALE); }
__device__ __forceinline__ float unfx(unsigned long long u) { return (float)(long long)u * FX_INV; }

__device__ __forceinline__ uint4 ldw16(const void* p) {   // streaming 16-byte load that never allocates in L1
  uint4 r;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
__device__ __forceinline__ void ldwv(const bf16* p, float* f) { unpack8(ldw16(p), f); }
__device__ __forceinline__ void ldwv(const float* p, float* f) {
  const uint4 u = ldw16(p); f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
}
template <class T> __device__ __forceinline__ float ldcg_f(const T* p);
template <> __device__ __forceinline__ float ldcg_f<bf16>(const bf16* p) { return __bfloat162float(__ldcg(p)); }
template <> __device__ __forceinline__ float ldcg_f<float>(const float* p) { return __ldcg(p); }

__device__ __forceinline__ bool better(float a, int ai, float b, int bi) {
  if (a != a) return false;
  if (b != b) return true;
  return a > b || (a == b && ai < bi);
}
__device__ __forceinline__ void block_argmax(float& v, int& idx, float* sv, int* si) {
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (better(ov, oi, v, idx)) { v = ov; idx = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) { sv[w] = v; si[w] = idx; }
  __syncthreads();
  v = sv[0]; idx = si[0];
#pragma unroll
  for (int i = 1; i < 8; i++) if (better(sv[i], si[i], v, idx)) { v = sv[i]; idx = si[i]; }
  __syncthreads();
}
// counter-based Gumbel(0,1) noise keyed by (seed, step, vocabulary index)
__device__ __forceinline__ float gumbel(u64 seed, uint32_t step, uint32_t v) {
  const u64 r = splitmix64(splitmix64(seed ^ ((u64)step << 32)) + v);
  const float u = ((float)(uint32_t)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);
  return -logf(-logf(u));
}

template <class T, int D, int DH> struct Geo {
  static constexpr int VN = Vec<T>::N;
  static constexpr int CB = D < 256 ? D : 256;        // residual columns per attention/Wo or down-projection pass
  static constexpr int NCB = D / CB;
  static constexpr int CG64 = 64 / VN;                // column groups of a 64-wide GEMV slice
  static constexpr int RG64 = NTHR / CG64;            // row groups
  static constexpr int CGB = CB / VN;                 // column groups of a CB-wide slice
  static constexpr int RGB = NTHR / CGB;
  static constexpr int LPK = DH / VN;                 // lanes per key row
  static constexpr int KPR = NTHR / LPK;              // keys per round
  static constexpr int RED = (RG64 * 64 > RGB * CB ? RG64 * 64 : RGB * CB) > KPR * DH ? (RG64 * 64 > RGB * CB ? RG64 * 64 : RGB * CB) : KPR * DH;
  static_assert(D % CB == 0 && D % 64 == 0 && DH % VN == 0 && NTHR % LPK == 0, "geometry");
};
// shared memory (floats): xs[D] | red[RED] | res[64] | scratch[32] | hb[64] | sc[T]
template <class T, int D, int DH> __host__ __device__ constexpr size_t smem_bytes(int Tctx) {
  return (size_t)(D + Geo<T, D, DH>::RED + 64 + 32 + 64 + Tctx + HR) * 4;
}

// xs[k] = round_T(LN(x)[k] * gamma[k]); x = fixed-point residual `src`. One block reduction of shifted sums.
template <class T, int D>
__device__ __forceinline__ void prologue_ln(const unsigned long long* src, const T* gamma, float* xs, float* scratch, unsigned long long* copy_to) {
  constexpr int NE = (D + NTHR - 1) / NTHR;
  const int tid = threadIdx.x;
  float x[NE], g[NE];
  const float xref = unfx(__ldcg(&src[0]));
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < NE; i++) {
    const int k = tid + i * NTHR;
    if (k < D) {
      const unsigned long long raw = __ldcg(&src[k]);
      g[i] = ldcg_f<T>(gamma + k);
      x[i] = unfx(raw);
      const float d = x[i] - xref;
      s1 += d; s2 += d * d;
      if (copy_to) copy_to[k] = raw;
    }
  }
  for (int o = 16; o; o >>= 1) { s1 += __shfl_xor_sync(0xffffffffu, s1, o); s2 += __shfl_xor_sync(0xffffffffu, s2, o); }
  if ((tid & 31) == 0) { scratch[tid >> 5] = s1; scratch[8 + (tid >> 5)] = s2; }
  __syncthreads();
  float t1 = 0.f, t2 = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) { t1 += scratch[i]; t2 += scratch[8 + i]; }
  const float m1 = t1 * (1.0f / D);
  const float var = fmaxf(t2 * (1.0f / D) - m1 * m1, 0.f);
  const float mean = xref + m1, rstd = rsqrtf(var + 1e-5f);
#pragma unroll
  for (int i = 0; i < NE; i++) {
    const int k = tid + i * NTHR;
    if (k < D) xs[k] = round_to<T>((x[i] - mean) * rstd * g[i]);
  }
  __syncthreads();
}

// res[c] = sum_{k<nk} xs[k] * W[k*ld + c0 + c], c in [0,64): thread (rg, cg) streams rows rg, rg+RG64, ... with 16-byte loads,
// UNR loads in flight; the RG64 partial sums of a column are added in index order. Ends with a sync (res valid).
template <class T, int D, int DH>
__device__ __forceinline__ void gemv64(const T* W, int ld, int c0, int nk, const float* xs, float* red, float* res) {
  using G = Geo<T, D, DH>;
  constexpr int VN = G::VN, UNR = 8;
  const int tid = threadIdx.x, rg = tid / G::CG64, cg = tid % G::CG64;
  float acc[VN];
#pragma unroll
  for (int i = 0; i < VN; i++) acc[i] = 0.f;
  const T* base = W + c0 + cg * VN;
  for (int k0 = rg; k0 < nk; k0 += G::RG64 * UNR) {
    float w[UNR][VN];
#pragma unroll
    for (int u = 0; u < UNR; u++) { const int k = k0 + u * G::RG64; if (k < nk) ldwv(base + (size_t)k * ld, w[u]); }
#pragma unroll
    for (int u = 0; u < UNR; u++) {
      const int k = k0 + u * G::RG64;
      if (k < nk) { const float x = xs[k];
#pragma unroll
        for (int i = 0; i < VN; i++) acc[i] += x * w[u][i]; }
    }
  }
#pragma unroll
  for (int i = 0; i < VN; i++) red[rg * 64 + cg * VN + i] = acc[i];
  __syncthreads();
  if (tid < 64) {
    float r = 0.f;
#pragma unroll 8
    for (int g = 0; g < G::RG64; g++) r += red[g * 64 + tid];
    res[tid] = r;
  }
  __syncthreads();
}

// out[c] += fixed(sum_{r<nr} h[r] * W[(r0+r)*D + cb*CB + c]) for c in [0,CB), added to up to two residual copies
template <class T, int D, int DH>
__device__ __forceinline__ void slice_to_residual(const T* W, int r0, int nr, int cb, const float* h, float* red,
                                                  unsigned long long* dst0, unsigned long long* dst1) {
  using G = Geo<T, D, DH>;
  constexpr int VN = G::VN;
  const int tid = threadIdx.x, rg = tid / G::CGB, cg = tid % G::CGB;
  float acc[VN];
#pragma unroll
  for (int i = 0; i < VN; i++) acc[i] = 0.f;
  for (int r = rg; r < nr; r += G::RGB) {
    float w[VN]; ldwv(W + (size_t)(r0 + r) * D + cb * G::CB + cg * VN, w);
    const float x = h[r];
#pragma unroll
    for (int i = 0; i < VN; i++) acc[i] += x * w[i];
  }
#pragma unroll
  for (int i = 0; i < VN; i++) red[rg * G::CB + cg * VN + i] = acc[i];
  __syncthreads();
  if (tid < G::CB) {
    float r = 0.f;
    for (int g = 0; g < G::RGB; g++) r += red[g * G::CB + tid];
    const unsigned long long u = fx(r);
    atomicAdd(&dst0[cb * G::CB + tid], u);
    if (dst1) atomicAdd(&dst1[cb * G::CB + tid], u);
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------------- tasks
// QKV: task t = columns [64t, 64t+64) of [q|k|v]; ntasks = 3D/64.
template <class T, int D, int DH>
__device__ __forceinline__ void task_qkv(const DecodeParams& P, const ModelDims& md, int layer, int t, unsigned char* smem) {
  using G = Geo<T, D, DH>;
  float* xs = reinterpret_cast<float*>(smem); float* red = xs + D; float* res = red + G::RED; float* scratch = res + 64;
  const DecodeState& st = P.st;
  prologue_ln<T, D>(st.xw, reinterpret_cast<const T*>(P.g1[layer]), xs, scratch, t == 0 ? st.xr : nullptr);
  gemv64<T, D, DH>(reinterpret_cast<const T*>(P.wqkv[layer]), 3 * D, t * 64, D, xs, red, res);
  if (threadIdx.x < 64) {
    const int col = t * 64 + threadIdx.x, which = col / D, within = col % D;
    const T o = from_f<T>(res[threadIdx.x]);
    if (which == 0) reinterpret_cast<T*>(st.q)[within] = o;
    else {
      const int head = within / DH, i = within % DH, pos = __ldcg(&st.scal[DS_POS]);
      reinterpret_cast<T*>(st.kv)[((((size_t)layer * 2 + (which - 1)) * md.H + head) * md.T + pos) * DH + i] = o;
    }
  }
}

// ATT+WO: task t -> head = t / NCB, column block cb = t % NCB; ntasks = H * NCB.
template <class T, int D, int DH>
__device__ __forceinline__ void task_attwo(const DecodeParams& P, const ModelDims& md, int layer, int t, unsigned char* smem) {
  using G = Geo<T, D, DH>;
  constexpr int VN = G::VN, LPK = G::LPK, KPR = G::KPR;
  float* xs = reinterpret_cast<float*>(smem); float* red = xs + D; float* res = red + G::RED; float* scratch = res + 64; float* ob = scratch + 32;
  float* sc = ob + 64;                                // [T]
  float* qs = xs;                                     // [DH]
  const DecodeState& st = P.st;
  const int tid = threadIdx.x, g = tid / LPK, l = tid % LPK;
  const int head = t / G::NCB, cb = t % G::NCB;
  const int n = __ldcg(&st.scal[DS_POS]) + 1;
  if (tid < DH) qs[tid] = ldcg_f<T>(reinterpret_cast<const T*>(st.q) + head * DH + tid) * rsqrtf((float)DH);
  __syncthreads();
  const T* Kc = reinterpret_cast<const T*>(st.kv) + (((size_t)layer * 2 + 0) * md.H + head) * md.T * DH;
  const T* Vc = reinterpret_cast<const T*>(st.kv) + (((size_t)layer * 2 + 1) * md.H + head) * md.T * DH;
  float qv[VN];
#pragma unroll
  for (int i = 0; i < VN; i++) qv[i] = qs[l * VN + i];
  constexpr int UK = 4;
  for (int jb = 0; jb < n; jb += KPR * UK) {
    float kw[UK][VN];
#pragma unroll
    for (int u = 0; u < UK; u++) { const int j = jb + g + KPR * u; ldwv(Kc + (size_t)(j < n ? j : 0) * DH + l * VN, kw[u]); }
#pragma unroll
    for (int u = 0; u < UK; u++) {
      const int j = jb + g + KPR * u;
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < VN; i++) d += qv[i] * kw[u][i];
#pragma unroll
      for (int o = 1; o < LPK; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (l == 0 && j < n) sc[j] = d;
    }
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int j = tid; j < n; j += NTHR) mx = fmaxf(mx, sc[j]);
  mx = block_max(mx, scratch);
  float sm = 0.f;
  for (int j = tid; j < n; j += NTHR) { const float e = expf(sc[j] - mx); sc[j] = e; sm += e; }
  sm = block_sum(sm, scratch);
  __syncthreads();
  float acc[VN];
#pragma unroll
  for (int i = 0; i < VN; i++) acc[i] = 0.f;
  for (int jb = 0; jb < n; jb += KPR * UK) {
    float vb[UK][VN];
#pragma unroll
    for (int u = 0; u < UK; u++) { const int j = jb + g + KPR * u; ldwv(Vc + (size_t)(j < n ? j : 0) * DH + l * VN, vb[u]); }
#pragma unroll
    for (int u = 0; u < UK; u++) {
      const int j = jb + g + KPR * u;
      if (j < n) { const float p = sc[j];
#pragma unroll
        for (int i = 0; i < VN; i++) acc[i] += p * vb[u][i]; }
    }
  }
#pragma unroll
  for (int i = 0; i < VN; i++) red[g * DH + l * VN + i] = acc[i];
  __syncthreads();
  if (tid < DH) {
    float o = 0.f;
    for (int gg = 0; gg < KPR; gg++) o += red[gg * DH + tid];
    ob[tid] = round_to<T>(o / sm);
  }
  __syncthreads();
  slice_to_residual<T, D, DH>(reinterpret_cast<const T*>(P.wo[layer]), head * DH, DH, cb, ob, red, st.xr, st.xw);
}

// UP+DOWN: task t = hidden units [64t, 64t+64); ntasks = FF/64.
template <class T, int D, int DH>
__device__ __forceinline__ void task_updn(const DecodeParams& P, const ModelDims& md, int layer, int t, unsigned char* smem) {
  using G = Geo<T, D, DH>;
  float* xs = reinterpret_cast<float*>(smem); float* red = xs + D; float* res = red + G::RED; float* scratch = res + 64; float* hb = scratch + 32;
  const DecodeState& st = P.st;
  prologue_ln<T, D>(st.xr, reinterpret_cast<const T*>(P.g2[layer]), xs, scratch, nullptr);
  gemv64<T, D, DH>(reinterpret_cast<const T*>(P.wup[layer]), md.FF, t * 64, D, xs, red, res);
  if (threadIdx.x < 64) hb[threadIdx.x] = round_to<T>(gelu_fwd<false>(res[threadIdx.x]));
  __syncthreads();
  for (int cb = 0; cb < G::NCB; cb++)
    slice_to_residual<T, D, DH>(reinterpret_cast<const T*>(P.wdn[layer]), t * 64, 64, cb, hb, red, st.xw, nullptr);
}

// HEAD: task t = vocabulary rows [128t, 128t+128); ntasks = ceil(V/128). Warp w streams rows 16w..16w+15, two at a time.
template <class T, int D, int DH>
__device__ __forceinline__ void task_head(const DecodeParams& P, const ModelDims& md, int t, unsigned char* smem) {
  using G = Geo<T, D, DH>;
  constexpr int VN = G::VN, VPR = D / VN, NCH = (VPR + 31) / 32, RPW = HR / 8;
  float* xs = reinterpret_cast<float*>(smem); float* red = xs + D; float* res = red + G::RED; float* scratch = res + 64;
  float* lg = scratch + 32 + 64 + md.T;               // [HR]
  const DecodeState& st = P.st;
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31;
  prologue_ln<T, D>(st.xw, reinterpret_cast<const T*>(P.gf), xs, scratch, nullptr);
  const T* Wh = reinterpret_cast<const T*>(P.head);
  for (int rb = 0; rb < RPW; rb += 2) {
    float s[2] = {0.f, 0.f};
    float wv[2][NCH][VN];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const int v = t * HR + w * RPW + rb + r;
#pragma unroll
      for (int i = 0; i < NCH; i++) { const int vi = lane + 32 * i; if (vi < VPR && v < md.V) ldwv(Wh + (size_t)v * D + vi * VN, wv[r][i]); }
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const int v = t * HR + w * RPW + rb + r;
#pragma unroll
      for (int i = 0; i < NCH; i++) {
        const int vi = lane + 32 * i;
        if (vi < VPR && v < md.V) {
#pragma unroll
          for (int k = 0; k < VN; k++) s[r] += xs[vi * VN + k] * wv[r][i][k];
        }
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) { s[0] += __shfl_xor_sync(0xffffffffu, s[0], o); s[1] += __shfl_xor_sync(0xffffffffu, s[1], o); }
    if (lane == 0) { lg[w * RPW + rb] = s[0]; lg[w * RPW + rb + 1] = s[1]; }
  }
  __syncthreads();
  float* sv = scratch; int* si = reinterpret_cast<int*>(scratch + 8);
  const float temp = P.temperature, invT = temp > 0.f ? 1.f / temp : 1.f;
  const uint32_t step = (uint32_t)__ldcg(&st.scal[DS_STEP]);
  const int nchunk = (md.V + HR - 1) / HR;
  float v0 = -INFINITY, v1 = -INFINITY;
  const int gi = t * HR + tid;
  if (tid < HR && gi < md.V) {
    const float l = lg[tid];
    st.logits[gi] = l;
    if (gi < md.valid_vocab) { v0 = l; v1 = temp > 0.f ? l * invT + gumbel(P.seed, step, gi) : l; }
  }
  float b0 = v0; int i0 = gi; block_argmax(b0, i0, sv, si);
  float b1 = v1; int i1 = gi; block_argmax(b1, i1, sv, si);
  if (tid == 0) { st.cand_v[t] = b0; st.cand_i[t] = i0; st.cand_v[nchunk + t] = b1; st.cand_i[nchunk + t] = i1; }
}

// xw := fixed point (wte[tok] + wpe[pos])
template <class T, int D>
__device__ __forceinline__ void write_embed(const DecodeParams& P, int tok, int pos) {
  for (int k = threadIdx.x; k < D; k += NTHR)
    P.st.xw[k] = fx(ldcg_f<T>(reinterpret_cast<const T*>(P.wte) + (size_t)tok * D + k) + ldcg_f<T>(reinterpret_cast<const T*>(P.wpe) + (size_t)pos * D + k));
}

// SAMPLE: one task. Final pick over the chunk candidates, prompt forcing / answer mode, pos/step update, next embedding.
template <class T, int D, int DH>
__device__ __forceinline__ void task_sample(const DecodeParams& P, const ModelDims& md, Live* live, unsigned char* smem) {
  const DecodeState& st = P.st;
  float* sv = reinterpret_cast<float*>(smem); int* si = reinterpret_cast<int*>(sv + 8); int* sn = si + 8;
  const int tid = threadIdx.x, mode = P.temperature > 0.f ? 1 : 0;
  const int nchunk = (md.V + HR - 1) / HR;
  float bv = -INFINITY; int bi = 0x7fffffff;
  for (int c = tid; c < nchunk; c += NTHR) {
    const float v = __ldcg(&st.cand_v[mode * nchunk + c]); const int i = __ldcg(&st.cand_i[mode * nchunk + c]);
    if (better(v, i, bv, bi)) { bv = v; bi = i; }
  }
  block_argmax(bv, bi, sv, si);
  if (tid == 0) {
    int step = st.scal[DS_STEP], pos = st.scal[DS_POS];
    int next = bi;
    if (P.answer_len > 0) {                            // answer mode: the prompt is fed again before every answer
      int astep = st.scal[DS_ASTEP];
      const bool forcing = astep + 1 < P.nforced;
      if (forcing) next = P.forced[astep + 1];
      if (st.out_tokens) st.out_tokens[step % st.out_cap] = forcing ? (astep == 0 ? OUT_RESTART : OUT_FORCED) : bi;
      pos += 1; astep += 1;
      if (astep >= P.nforced - 1 + P.answer_len) { next = P.forced[0]; pos = 0; astep = 0; }
      st.scal[DS_ASTEP] = astep;
    } else {
      if (step + 1 < P.nforced) next = P.forced[step + 1];
      if (st.out_tokens) st.out_tokens[step % st.out_cap] = bi;
      pos += 1;
    }
    st.scal[DS_CTXFULL] = (pos >= md.T);
    if (pos >= md.T && P.auto_reset) pos = 0;
    st.scal[DS_TOKEN] = next; st.scal[DS_POS] = pos; st.scal[DS_STEP] = step + 1;
    if (live) live->dec_steps = (unsigned)(step + 1);
    sn[0] = next; sn[1] = pos;
  }
  __syncthreads();
  write_embed<T, D>(P, sn[0], sn[1]);
}

}  // namespace dec
}  // namespace ofa
