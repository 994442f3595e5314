// Batch-1 KV-cache decode from the LIVE working-copy weights, as tasks of the serving job.
//
// Phase structure and every rounding point follow the reference's decode task set
// (llm/b200/megakernel/decode_wide.cuh:251-626): per layer QKV (LN1 prologue + 64-column GEMV slice, K/V row appended at
// `pos`), ATT+WO (one head's softmax attention + its slice of Wo), UP+DOWN (LN2 + 32 hidden units + their slice of Wdown);
// then HEAD (LN_f + 64 vocabulary rows per task, fp32 logits, chunk-local argmax / Gumbel-max) and SAMPLE (fixed-order
// final pick, prompt forcing / answer mode, position update, next embedding). The residual stream is kept in int64 fixed
// point (2^-30 units) and updated with integer atomics, so the result is bitwise independent of task order. LN output,
// attention output and GELU output are each rounded to the activation type T before the next product; q, K, V are stored
// as T; softmax uses expf; GELU uses tanhf; argmax ties go to the lower index and NaN never wins.
// Nothing synchronises the decoder with the trainer: it reads whatever the working copy holds.
//
// What is different from the reference is where the weights wait. A serving block knows its next task as soon as it has
// claimed the ticket, usually before the task's dependencies are complete. In that window it starts bulk copies (TMA,
// cp.async.bulk, completion counted on an mbarrier) of everything the task will read that does not depend on the current
// token - its weight slice, and for attention the K/V rows of earlier positions - into a 96 KB shared-memory buffer. When the
// dependencies resolve the task only runs its LayerNorm prologue and multiplies out of shared memory, so the 38 dependent
// phases of a token no longer each pay a DRAM round trip (measured before this change: 5 us of an 8.7 us QKV task was
// waiting for its second batch of weight loads).
//
// Unlike the reference, the code is generic over T in {bf16, float}, the width D and the head dim DH (the thread mappings
// are derived from the 16-byte vector width), so the tiny fp32 model runs through the same tasks.
#pragma once
#include "common.cuh"
#include "task_api.h"

namespace ofa {
namespace dec {

constexpr int HR = 64;                                // vocabulary rows per head task (one task's rows fill the weight buffer)
constexpr int HU = 32;                                // hidden units per UP+DOWN task
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
template <class T> __device__ __forceinline__ void cvt16(uint4 u, float* f);      // 16 raw bytes -> Vec<T>::N floats
template <> __device__ __forceinline__ void cvt16<bf16>(uint4 u, float* f) { unpack8(u, f); }
template <> __device__ __forceinline__ void cvt16<float>(uint4 u, float* f) { f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w); }
template <class T> __device__ __forceinline__ float ldcg_f(const T* p);
template <> __device__ __forceinline__ float ldcg_f<bf16>(const bf16* p) { return __bfloat162float(__ldcg(p)); }
template <> __device__ __forceinline__ float ldcg_f<float>(const float* p) { return __ldcg(p); }

// L2 prefetch of part `part` of `nparts` of a contiguous byte range (128-byte lines), spread over the 256 threads. Weights do
// not depend on activations, so every decode task pulls a share of the NEXT phase's weights towards L2 before it starts its
// own dependent work; the next phase then streams from L2 instead of DRAM. Hint only: it never changes results.
__device__ __forceinline__ void l2_prefetch_share(const void* base, size_t bytes, int part, int nparts) {
  const size_t lines = (bytes + 127) >> 7;
  const size_t per = (lines + nparts - 1) / nparts;
  const size_t lo = per * part, hi = lo + per < lines ? lo + per : lines;
  const char* b = reinterpret_cast<const char*>(base);
  for (size_t i = lo + threadIdx.x; i < hi; i += NTHR) asm volatile("prefetch.global.L2 [%0];" ::"l"(b + (i << 7)));
}

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

// stage stamps of one traced task instance (layer 0, task 0): slot base + i
__device__ __forceinline__ void trace(unsigned long long* tr, bool on, int slot) { if (on && tr && threadIdx.x == 0) tr[slot] = gtimer(); }

template <class T, int D, int DH> struct Geo {
  static constexpr int VN = Vec<T>::N;
  static constexpr int ES = (int)sizeof(T);
  static constexpr int CB = D < 256 ? D : 256;        // residual columns per attention/Wo task
  static constexpr int NCB = D / CB;
  static constexpr int WB = D * 64 * ES;              // weight buffer: one 64-column slice of a [D, *] matrix (98,304 B for GPT-S)
  static constexpr int WO_BYTES = DH * CB * ES;       // Wo slice of an attention task
  static constexpr int KV_ROWS = (WB - WO_BYTES) / 2 / (DH * ES);   // K (and V) rows of earlier positions that fit beside it
  static constexpr int LPK = DH / VN;                 // lanes per key row
  static constexpr int KPR = NTHR / LPK;              // keys per round
  static constexpr int RED = 1024;                    // floats of reduction scratch
  static_assert(D % CB == 0 && D % 64 == 0 && DH % VN == 0 && NTHR % LPK == 0 && HU * D * ES * 2 <= WB && HR * D * ES <= WB && KPR * DH <= 2048, "geometry");
};
// shared memory: weight buffer [WB] | floats xs[D] red[2048] res[64] scratch[32] hb[64] sc[T] lg[HR] | int meta[4]
template <class T, int D, int DH> __host__ __device__ constexpr size_t smem_bytes(int Tctx) {
  return (size_t)Geo<T, D, DH>::WB + (size_t)(D + 2048 + 64 + 32 + 64 + Tctx + HR + 4) * 4;
}
template <class T, int D, int DH> struct Smem {
  unsigned char* w; float *xs, *red, *res, *scratch, *hb, *sc, *lg; int* meta;
  __device__ __forceinline__ Smem(unsigned char* base, int Tctx) {
    w = base; xs = reinterpret_cast<float*>(base + Geo<T, D, DH>::WB); red = xs + D; res = red + 2048; scratch = res + 64; hb = scratch + 32;
    sc = hb + 64; lg = sc + Tctx; meta = reinterpret_cast<int*>(lg + HR);
  }
};

// once per serving block, before its first task
template <class T, int D, int DH>
__device__ __forceinline__ void block_init(unsigned char* smem, int Tctx) {
  Smem<T, D, DH> S(smem, Tctx);
  if (threadIdx.x < 4) S.meta[threadIdx.x] = 0;
}

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void ld2(const bf16* p, float& a, float& b) { const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); a = f.x; b = f.y; }
__device__ __forceinline__ void ld2(const float* p, float& a, float& b) { const float2 f = *reinterpret_cast<const float2*>(p); a = f.x; b = f.y; }

// ---------------------------------------------------------------------------------------------- prefetch (runs while the task's dependencies are still pending)
// Starts the bulk copies of task (kind, layer, t) into the weight buffer; warp 0 only. Returns true (uniformly for the block)
// if the task has a fill to wait for. `bar` is the block's fill barrier (count 1); each fill is one phase of it.
template <class T, int D, int DH>
__device__ __forceinline__ bool prefetch(const DecodeParams& P, const ModelDims& md, int kind, int layer, int t, unsigned char* smem, uint32_t bar) {
  using G = Geo<T, D, DH>;
  if (kind == TK_DEC_SAMPLE) return false;
  if (threadIdx.x >= 32) return true;
  const int lane = threadIdx.x;
  const uint32_t dst = smem_u32(smem);
  Smem<T, D, DH> S(smem, md.T);
  fence_proxy_async();          // the previous task's ordinary accesses to the buffer come before these asynchronous writes
  switch (kind) {
    case TK_DEC_QKV: {
      constexpr int RBY = 64 * G::ES;
      if (lane == 0) mbar_expect_tx(bar, D * RBY);
      __syncwarp();
      constexpr int BR = D < 256 ? D : 256;            // rows per TMA box
      if (lane < D / BR) tma_load_2d(dst + lane * BR * RBY, reinterpret_cast<const char*>(P.tm_qkv) + (size_t)layer * 128, bar, t * 64, lane * BR);
      break;
    }
    case TK_DEC_ATTWO: {
      const int head = t / G::NCB, cb = t % G::NCB;
      // rows of earlier positions: the position word may be older than the token this task belongs to (tickets are claimed
      // ahead), so the epoch it carries is kept and the task uses the copied rows only if it runs in the same context
      const int key = __ldcg(&P.st.scal[DS_POSKEY]);
      int np = key & 0xFFFF;
      np = np < G::KV_ROWS ? np : G::KV_ROWS;
      const uint32_t kvb = (uint32_t)np * DH * G::ES;
      if (lane == 0) { S.meta[0] = np; S.meta[1] = key >> 16; mbar_expect_tx(bar, G::WO_BYTES + 2 * kvb); }
      __syncwarp();
      if (lane == 2) tma_load_2d(dst, reinterpret_cast<const char*>(P.tm_wo) + (size_t)layer * 128, bar, cb * G::CB, head * DH);
      if (np > 0 && lane < 2) {
        const T* kv = reinterpret_cast<const T*>(P.st.kv) + (((size_t)layer * 2 + lane) * md.H + head) * md.T * DH;
        bulk_g2s(dst + G::WO_BYTES + lane * G::KV_ROWS * DH * G::ES, kv, kvb, bar);
      }
      break;
    }
    case TK_DEC_UPDN: {
      constexpr int RBY = HU * G::ES;
      if (lane == 0) mbar_expect_tx(bar, 2 * D * RBY);
      __syncwarp();
      constexpr int BR = D < 256 ? D : 256;
      if (lane >= 1 && lane <= D / BR) tma_load_2d(dst + (lane - 1) * BR * RBY, reinterpret_cast<const char*>(P.tm_up) + (size_t)layer * 128, bar, t * HU, (lane - 1) * BR);
      if (lane == 0) bulk_g2s(dst + D * RBY, reinterpret_cast<const T*>(P.wdn[layer]) + (size_t)t * HU * D, D * RBY, bar);
      break;
    }
    default: {  // TK_DEC_HEAD
      const int rows = min(HR, md.V - t * HR);
      if (lane == 0) { mbar_expect_tx(bar, rows * D * G::ES); bulk_g2s(dst, reinterpret_cast<const T*>(P.head) + (size_t)t * HR * D, rows * D * G::ES, bar); }
      break;
    }
  }
  return true;
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

// res[c] = sum_k xs[k] * W[k][c] for a [nk][NC] slice resident in shared memory (NC = 64 or 32). Thread = (row group, column
// pair); the row-group partials of a column are added in index order. Ends with a sync (res valid).
template <class T, int NC>
__device__ __forceinline__ void gemv_smem(const T* W, int nk, const float* xs, float* red, float* res) {
  constexpr int CP = NC / 2, RG = NTHR / CP;
  const int tid = threadIdx.x, cp = tid % CP, rg = tid / CP;
  float a0 = 0.f, a1 = 0.f;
#pragma unroll 4
  for (int k = rg; k < nk; k += RG) {
    float w0, w1; ld2(W + (size_t)k * NC + 2 * cp, w0, w1);
    const float x = xs[k];
    a0 += x * w0; a1 += x * w1;
  }
  red[rg * NC + 2 * cp] = a0; red[rg * NC + 2 * cp + 1] = a1;
  __syncthreads();
  if (tid < NC) {
    float r = 0.f;
#pragma unroll 8
    for (int g = 0; g < RG; g++) r += red[g * NC + tid];
    res[tid] = r;
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------------- tasks
// Every task: dependent prologue first, then wait (bounded) for its fill, then multiply out of shared memory.
#define OFA_DEC_WAIT_FILL()                                                                                        \
  {                                                                                                                 \
    const bool ok_ = mbar_wait(bar, parity, status);                                                                \
    if (!ok_ && !aborted(status)) raise_abort(status, ST_MBAR_FULL_TIMEOUT, -2, t, layer);                          \
    if (__syncthreads_or(!ok_)) return;      /* uniform decision: nobody is left behind at a later barrier */       \
  }

// QKV: task t = columns [64t, 64t+64) of [q|k|v]; ntasks = 3D/64.
template <class T, int D, int DH>
__device__ __forceinline__ void task_qkv(const DecodeParams& P, const ModelDims& md, int layer, int t, unsigned char* smem, uint32_t bar, uint32_t parity, DevStatus* status) {
  Smem<T, D, DH> S(smem, md.T);
  const DecodeState& st = P.st;
  const bool tr = layer == 0 && t == 0;
  trace(P.trace, tr, 0);
  if (threadIdx.x == 0) S.meta[2] = 0;                 // xs no longer holds a final-LayerNorm row
  prologue_ln<T, D>(st.xw, reinterpret_cast<const T*>(P.g1[layer]), S.xs, S.scratch, t == 0 ? st.xr : nullptr);
  trace(P.trace, tr, 1);
  OFA_DEC_WAIT_FILL();
  trace(P.trace, tr, 2);
  gemv_smem<T, 64>(reinterpret_cast<const T*>(S.w), D, S.xs, S.red, S.res);
  trace(P.trace, tr, 3);
  if (threadIdx.x < 64) {
    const int col = t * 64 + threadIdx.x, which = col / D, within = col % D;
    const T o = from_f<T>(S.res[threadIdx.x]);
    if (which == 0) reinterpret_cast<T*>(st.q)[within] = o;
    else {
      const int head = within / DH, i = within % DH, pos = __ldcg(&st.scal[DS_POS]);
      reinterpret_cast<T*>(st.kv)[((((size_t)layer * 2 + (which - 1)) * md.H + head) * md.T + pos) * DH + i] = o;
    }
  }
  trace(P.trace, tr, 4);
}

// ATT+WO: task t -> head = t / NCB, column block cb = t % NCB; ntasks = H * NCB. K/V rows below min(prefetched, pos) come from
// shared memory, the rest (at least the current token's row) from global memory.
template <class T, int D, int DH>
__device__ __forceinline__ void task_attwo(const DecodeParams& P, const ModelDims& md, int layer, int t, unsigned char* smem, uint32_t bar, uint32_t parity, DevStatus* status) {
  using G = Geo<T, D, DH>;
  constexpr int VN = G::VN, LPK = G::LPK, KPR = G::KPR;
  Smem<T, D, DH> S(smem, md.T);
  float* qs = S.xs;                                   // [DH]
  float* ob = S.hb;
  const DecodeState& st = P.st;
  const int tid = threadIdx.x, g = tid / LPK, l = tid % LPK;
  const int head = t / G::NCB, cb = t % G::NCB;
  const int pos = __ldcg(&st.scal[DS_POS]), n = pos + 1;
  if (tid == 0) S.meta[2] = 0;
  if (tid < DH) qs[tid] = ldcg_f<T>(reinterpret_cast<const T*>(st.q) + head * DH + tid) * rsqrtf((float)DH);
  OFA_DEC_WAIT_FILL();
  const int nres = (S.meta[1] == (__ldcg(&st.scal[DS_POSKEY]) >> 16)) ? min(S.meta[0], pos) : 0;   // rows valid in shared memory
  const T* Kc = reinterpret_cast<const T*>(st.kv) + (((size_t)layer * 2 + 0) * md.H + head) * md.T * DH;
  const T* Vc = reinterpret_cast<const T*>(st.kv) + (((size_t)layer * 2 + 1) * md.H + head) * md.T * DH;
  const T* sK = reinterpret_cast<const T*>(S.w + G::WO_BYTES);
  const T* sV = sK + (size_t)G::KV_ROWS * DH;
  float qv[VN];
#pragma unroll
  for (int i = 0; i < VN; i++) qv[i] = qs[l * VN + i];
  constexpr int UK = 4;
  for (int jb = 0; jb < n; jb += KPR * UK) {
    uint4 kw[UK];
#pragma unroll
    for (int u = 0; u < UK; u++) {
      const int j = jb + g + KPR * u;
      if (j < nres) kw[u] = *reinterpret_cast<const uint4*>(sK + (size_t)j * DH + l * VN);
      else kw[u] = ldw16(Kc + (size_t)(j < n ? j : 0) * DH + l * VN);
    }
#pragma unroll
    for (int u = 0; u < UK; u++) {
      const int j = jb + g + KPR * u;
      float f[VN]; cvt16<T>(kw[u], f);
      float d = 0.f;
#pragma unroll
      for (int i = 0; i < VN; i++) d += qv[i] * f[i];
#pragma unroll
      for (int o = 1; o < LPK; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      if (l == 0 && j < n) S.sc[j] = d;
    }
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int j = tid; j < n; j += NTHR) mx = fmaxf(mx, S.sc[j]);
  mx = block_max(mx, S.scratch);
  float sm = 0.f;
  for (int j = tid; j < n; j += NTHR) { const float e = expf(S.sc[j] - mx); S.sc[j] = e; sm += e; }
  sm = block_sum(sm, S.scratch);
  __syncthreads();
  float acc[VN];
#pragma unroll
  for (int i = 0; i < VN; i++) acc[i] = 0.f;
  for (int jb = 0; jb < n; jb += KPR * UK) {
    uint4 vb[UK];
#pragma unroll
    for (int u = 0; u < UK; u++) {
      const int j = jb + g + KPR * u;
      if (j < nres) vb[u] = *reinterpret_cast<const uint4*>(sV + (size_t)j * DH + l * VN);
      else vb[u] = ldw16(Vc + (size_t)(j < n ? j : 0) * DH + l * VN);
    }
#pragma unroll
    for (int u = 0; u < UK; u++) {
      const int j = jb + g + KPR * u;
      if (j < n) {
        const float p = S.sc[j];
        float f[VN]; cvt16<T>(vb[u], f);
#pragma unroll
        for (int i = 0; i < VN; i++) acc[i] += p * f[i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < VN; i++) S.red[g * DH + l * VN + i] = acc[i];
  __syncthreads();
  if (tid < DH) {
    float o = 0.f;
    for (int gg = 0; gg < KPR; gg++) o += S.red[gg * DH + tid];
    ob[tid] = round_to<T>(o / sm);
  }
  __syncthreads();
  if (tid < G::CB) {                                   // o[DH] . Wo slice: one column per thread, rows in order, no reduction
    const T* W = reinterpret_cast<const T*>(S.w);
    float r = 0.f;
#pragma unroll 8
    for (int k = 0; k < DH; k++) r += ob[k] * to_f(W[k * G::CB + tid]);
    const unsigned long long u = fx(r);
    atomicAdd(&st.xr[cb * G::CB + tid], u);
    atomicAdd(&st.xw[cb * G::CB + tid], u);
  }
}

// UP+DOWN: task t = hidden units [32t, 32t+32); ntasks = FF/32.
template <class T, int D, int DH>
__device__ __forceinline__ void task_updn(const DecodeParams& P, const ModelDims& md, int layer, int t, unsigned char* smem, uint32_t bar, uint32_t parity, DevStatus* status) {
  using G = Geo<T, D, DH>;
  Smem<T, D, DH> S(smem, md.T);
  const DecodeState& st = P.st;
  const bool tr = layer == 0 && t == 0;
  trace(P.trace, tr, 8);
  if (threadIdx.x == 0) S.meta[2] = 0;
  prologue_ln<T, D>(st.xr, reinterpret_cast<const T*>(P.g2[layer]), S.xs, S.scratch, nullptr);
  trace(P.trace, tr, 9);
  OFA_DEC_WAIT_FILL();
  trace(P.trace, tr, 10);
  gemv_smem<T, HU>(reinterpret_cast<const T*>(S.w), D, S.xs, S.red, S.res);
  trace(P.trace, tr, 11);
  if (threadIdx.x < HU) S.hb[threadIdx.x] = round_to<T>(gelu_fwd<false>(S.res[threadIdx.x]));
  __syncthreads();
  const T* Wd = reinterpret_cast<const T*>(S.w + (size_t)D * HU * G::ES);      // [HU][D]
  for (int c = threadIdx.x; c < D; c += NTHR) {
    float r = 0.f;
#pragma unroll 8
    for (int k = 0; k < HU; k++) r += S.hb[k] * to_f(Wd[k * D + c]);
    atomicAdd(&st.xw[c], fx(r));
  }
  trace(P.trace, tr, 12);
}

// HEAD: task t = vocabulary rows [64t, 64t+64); ntasks = ceil(V/64). Warp w owns rows 8w..8w+7.
template <class T, int D, int DH>
__device__ __forceinline__ void task_head(const DecodeParams& P, const ModelDims& md, int t, unsigned char* smem, uint32_t bar, uint32_t parity, DevStatus* status) {
  using G = Geo<T, D, DH>;
  constexpr int VN = G::VN, VPR = D / VN, NCH = (VPR + 31) / 32, RPW = HR / 8;
  Smem<T, D, DH> S(smem, md.T);
  const DecodeState& st = P.st;
  const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, layer = -1;
  // the final LayerNorm is the same for every head task of a token: a block that runs several of them in a row keeps it
  const int tag = __ldcg(&st.scal[DS_STEP]) + 1;
  if (S.meta[2] != tag) {
    prologue_ln<T, D>(st.xw, reinterpret_cast<const T*>(P.gf), S.xs, S.scratch, nullptr);
    if (tid == 0) S.meta[2] = tag;
  }
  OFA_DEC_WAIT_FILL();
  const T* Wh = reinterpret_cast<const T*>(S.w);
#pragma unroll 2
  for (int rr = 0; rr < RPW; rr++) {
    const int row = w * RPW + rr, v = t * HR + row;
    float s = 0.f;
    if (v < md.V) {
#pragma unroll
      for (int i = 0; i < NCH; i++) {
        const int vi = lane + 32 * i;
        if (vi < VPR) {
          float f[VN]; cvt16<T>(*reinterpret_cast<const uint4*>(Wh + (size_t)row * D + vi * VN), f);
#pragma unroll
          for (int k = 0; k < VN; k++) s += S.xs[vi * VN + k] * f[k];
        }
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) S.lg[row] = s;
  }
  __syncthreads();
  float* sv = S.scratch; int* si = reinterpret_cast<int*>(S.scratch + 8);
  const float temp = P.temperature, invT = temp > 0.f ? 1.f / temp : 1.f;
  const uint32_t step = (uint32_t)__ldcg(&st.scal[DS_STEP]);
  const int nchunk = (md.V + HR - 1) / HR;
  float v0 = -INFINITY, v1 = -INFINITY;
  const int gi = t * HR + tid;
  if (tid < HR && gi < md.V) {
    const float l = S.lg[tid];
    st.logits[gi] = l;
    if (gi < md.valid_vocab) { v0 = l; v1 = temp > 0.f ? l * invT + gumbel(P.seed, step, gi) : l; }
  }
  float b0 = v0; int i0 = gi; block_argmax(b0, i0, sv, si);
  float b1 = b0; int i1 = i0;
  if (temp > 0.f) { b1 = v1; i1 = gi; block_argmax(b1, i1, sv, si); }
  if (tid == 0) { st.cand_v[t] = b0; st.cand_i[t] = i0; st.cand_v[nchunk + t] = b1; st.cand_i[nchunk + t] = i1; }
}
#undef OFA_DEC_WAIT_FILL

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
    int epoch = st.scal[DS_EPOCH];
    if (pos == 0) { epoch = (epoch + 1) & 0x7FFF; st.scal[DS_EPOCH] = epoch; }      // a new context starts
    st.scal[DS_POSKEY] = (epoch << 16) | pos;
    st.scal[DS_TOKEN] = next; st.scal[DS_POS] = pos; st.scal[DS_STEP] = step + 1;
    if (live) live->dec_steps = (unsigned)(step + 1);
    sn[0] = next; sn[1] = pos;
  }
  __syncthreads();
  write_embed<T, D>(P, sn[0], sn[1]);
}

}  // namespace dec
}  // namespace ofa
