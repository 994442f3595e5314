// Memory-bound training tasks: embedding forward/backward, LayerNorm forward/backward (+dgamma reduce), softmax
// cross-entropy with in-place dlogits, mean loss, and the fused AdamW. Every task is templated on the activation storage
// type T (bf16 for GPT-S, float for the tiny model) and, where a row lives in registers, on the model width D.
//
// Semantics follow the reference task libraries (llm/elementwise/ew_layernorm.cuh:12-173, ew_loss.cuh:19-192,
// ew_adamw.cuh:20-67): fp32 statistics, gamma-only LayerNorm with eps 1e-5, two-pass variance, cross-entropy in the exp2
// domain over the STORED (rounded) logits with dlogits = (softmax - onehot)/N written over the logits, deterministic
// embedding scatter (contributions added in increasing token index), AdamW with torch's operation order. All reductions
// have a fixed order, so results do not depend on which block runs which task.
//
// Gradient buffers are OVERWRITTEN by their single producer each step (accumulate flags exist for the tied-head case),
// so AdamW neither reads stale sums nor has to zero the gradient buffer afterwards.
#pragma once
#include "common.cuh"
#include "task_api.h"

namespace ofa {
namespace ew {

constexpr int ROWS_PER_TASK = 16;    // embed / LayerNorm granularity
constexpr int CE_ROWS = 4;           // rows per cross-entropy task
constexpr int EMB_VCHUNK = 128;      // vocabulary rows per embedding-backward task
constexpr int OPT_CHUNK = 65536;     // elements per AdamW task
constexpr int WPE_ROWS = 4;          // positions per wpe-backward task
constexpr int SUM_CHUNK = 16384;     // elements per split-K reduce task

// global -> shared bulk copy by the copy engine (16-byte aligned addresses, size a multiple of 16), completion counted in bytes on `bar`
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void ld4(const float* p, float* f) { ldv(p, f); }
__device__ __forceinline__ void ld4(const bf16* p, float* f) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
  f[0] = __bfloat162float(a.x); f[1] = __bfloat162float(a.y); f[2] = __bfloat162float(b.x); f[3] = __bfloat162float(b.y);
}
__device__ __forceinline__ void st4(float* p, const float* f) { stv(p, f); }
__device__ __forceinline__ void st4(bf16* p, const float* f) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  uint2 u; u.x = *reinterpret_cast<const uint32_t*>(&a); u.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

// ---------------------------------------------------------------------------------------------- embedding forward
// x[r,:] = T(float(wte[tok[r],:]) + float(wpe[r % Tctx,:]));  task = 16 rows.
template <class T, int D>
__device__ __forceinline__ void embed_fwd_task(int task, T* x, const T* wte, const T* wpe, const int* tok, int N, int Tctx) {
  constexpr int VN = Vec<T>::N, VPR = D / VN;
  static_assert(D % VN == 0, "row must be a whole number of 16-byte vectors");
  const int r0 = task * ROWS_PER_TASK;
  for (int i = threadIdx.x; i < ROWS_PER_TASK * VPR; i += NTHR) {
    const int r = r0 + i / VPR;
    if (r >= N) break;
    const int c = (i % VPR) * VN;
    float a[VN], b[VN];
    ldv(wte + (size_t)tok[r] * D + c, a);
    ldv(wpe + (size_t)(r % Tctx) * D + c, b);
#pragma unroll
    for (int k = 0; k < VN; k++) a[k] += b[k];
    stv(x + (size_t)r * D + c, a);
  }
}

// ---------------------------------------------------------------------------------------------- LayerNorm
// Task = 16 rows, two per warp. A task is a handful of microseconds long and latency-bound (16 resident warps per SM, every
// load a round trip to L2 or HBM), so both rows of a warp are FETCHED before anything is computed: a lane keeps its share of a
// row as raw 16-byte vectors (vectors lane, lane+32, ... of the row) and converts them when it needs them, which keeps two
// rows (and for the backward task two operands per row) in flight at a time without running out of registers.
// Semantics are the reference's (llm/elementwise/ew_layernorm.cuh:38-173): gamma only, eps 1e-5, fp32 statistics, two-pass
// variance; backward dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) [+ dres] with g = dy * gamma.
template <class T, int D> struct RowRegs {
  static constexpr int VN = Vec<T>::N;
  static constexpr int VPR = D / VN;                 // vectors per row
  static constexpr int NV = (VPR + 31) / 32;         // vectors per lane
};
template <class T, int D> struct RowShare {          // one lane's share of one row, raw
  using R = RowRegs<T, D>;
  uint4 raw[R::NV];
  __device__ __forceinline__ void fetch(const T* row, int lane) {
#pragma unroll
    for (int v = 0; v < R::NV; v++) {
      const int vi = v * 32 + lane;
      raw[v] = vi < R::VPR ? *reinterpret_cast<const uint4*>(row + vi * R::VN) : make_uint4(0, 0, 0, 0);
    }
  }
  __device__ __forceinline__ void get(int v, float* f) const {
    if constexpr (sizeof(T) == 2) unpack8(raw[v], f);
    else { f[0] = __uint_as_float(raw[v].x); f[1] = __uint_as_float(raw[v].y); f[2] = __uint_as_float(raw[v].z); f[3] = __uint_as_float(raw[v].w); }
  }
  static __device__ __forceinline__ bool has(int v, int lane) { return v * 32 + lane < R::VPR; }
};
// two independent butterfly sums at once (the shuffles of one hide behind the other's)
__device__ __forceinline__ void warp_sum2(float& a, float& b) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
}

// y = (x - mean) * rstd * gamma, saves mean / rstd. Warp w: rows w and w + 8 of the task.
template <class T, int D>
__device__ __noinline__ void ln_fwd_task(int task, T* y, float* mean_o, float* rstd_o, const T* x, const T* gamma, int N) {
  using R = RowRegs<T, D>;
  using S = RowShare<T, D>;
  constexpr int VN = R::VN, NV = R::NV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row[2] = {task * ROWS_PER_TASK + warp, task * ROWS_PER_TASK + warp + 8};
  S in[2], gm;
#pragma unroll
  for (int j = 0; j < 2; j++) if (row[j] < N) in[j].fetch(x + (size_t)row[j] * D, lane);
  gm.fetch(gamma, lane);
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 2; j++)
    if (row[j] < N) {
#pragma unroll
      for (int v = 0; v < NV; v++) { float f[VN]; in[j].get(v, f);
#pragma unroll
        for (int k = 0; k < VN; k++) sum[j] += f[k]; }     // absent vectors are zero
    }
  warp_sum2(sum[0], sum[1]);
  const float mean[2] = {sum[0] * (1.f / D), sum[1] * (1.f / D)};
  float sq[2] = {0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 2; j++)
    if (row[j] < N) {
#pragma unroll
      for (int v = 0; v < NV; v++)
        if (S::has(v, lane)) { float f[VN]; in[j].get(v, f);
#pragma unroll
          for (int k = 0; k < VN; k++) { const float d = f[k] - mean[j]; sq[j] += d * d; } }
    }
  warp_sum2(sq[0], sq[1]);
#pragma unroll
  for (int j = 0; j < 2; j++) {
    if (row[j] >= N) continue;
    const float rstd = rsqrtf(sq[j] * (1.f / D) + 1e-5f);
#pragma unroll
    for (int v = 0; v < NV; v++)
      if (S::has(v, lane)) {
        float f[VN], g[VN];
        in[j].get(v, f); gm.get(v, g);
#pragma unroll
        for (int k = 0; k < VN; k++) f[k] = (f[k] - mean[j]) * rstd * g[k];
        stv(y + (size_t)row[j] * D + (v * 32 + lane) * VN, f);
      }
    if (lane == 0) { mean_o[row[j]] = mean[j]; rstd_o[row[j]] = rstd; }
  }
}

template <int D> __host__ __device__ constexpr size_t ln_bwd_smem_bytes() { return 8 * (size_t)D * sizeof(float); }

// dx, and this task's dgamma partial [task, D] = sum over its rows of dy * xhat (the eight warps' shares added in warp order).
// A row's three operands (x, dy, dres) are fetched together before anything is computed; pass 1 forms the two row sums and
// the dgamma terms, pass 2 recomputes xhat and g from the raw vectors (a few FMAs) instead of keeping them. The two rows of a
// warp go one after the other: with both in flight the persistent kernel's 128-register budget spilled.
template <class T, int D>
__device__ __noinline__ void ln_bwd_task(int task, T* dx, float* dgamma_part, const T* dy, const T* x, const float* mean,
                                            const float* rstd, const T* gamma, const T* dres, int N, unsigned char* smem) {
  using R = RowRegs<T, D>;
  using S = RowShare<T, D>;
  constexpr int VN = R::VN, NV = R::NV;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* sdg = reinterpret_cast<float*>(smem);   // [8][D]
  S gm;
  gm.fetch(gamma, lane);
  float dg[NV][VN];
#pragma unroll
  for (int v = 0; v < NV; v++)
#pragma unroll
    for (int k = 0; k < VN; k++) dg[v][k] = 0.f;
#pragma unroll 1
  for (int j = 0; j < 2; j++) {
    const int r = task * ROWS_PER_TASK + warp + j * 8;
    if (r >= N) continue;
    S xin, gin, res;
    xin.fetch(x + (size_t)r * D, lane); gin.fetch(dy + (size_t)r * D, lane);
    if (dres) res.fetch(dres + (size_t)r * D, lane);
    const float mu = mean[r], rs = rstd[r];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; v++)
      if (S::has(v, lane)) {
        float xv[VN], dv[VN], gv[VN];
        xin.get(v, xv); gin.get(v, dv); gm.get(v, gv);
#pragma unroll
        for (int k = 0; k < VN; k++) {
          const float xh = (xv[k] - mu) * rs, g = dv[k] * gv[k];
          s1 += g; s2 += g * xh;
          dg[v][k] += dv[k] * xh;
        }
      }
    warp_sum2(s1, s2);
    const float m1 = s1 * (1.f / D), m2 = s2 * (1.f / D);
#pragma unroll
    for (int v = 0; v < NV; v++)
      if (S::has(v, lane)) {
        float xv[VN], dv[VN], gv[VN], o[VN];
        xin.get(v, xv); gin.get(v, dv); gm.get(v, gv);
#pragma unroll
        for (int k = 0; k < VN; k++) { const float xh = (xv[k] - mu) * rs; o[k] = rs * (dv[k] * gv[k] - m1 - xh * m2); }
        if (dres) { float e[VN]; res.get(v, e);
#pragma unroll
          for (int k = 0; k < VN; k++) o[k] += e[k]; }
        stv(dx + (size_t)r * D + (v * 32 + lane) * VN, o);
      }
  }
#pragma unroll
  for (int v = 0; v < NV; v++)
    if (S::has(v, lane)) {
#pragma unroll
      for (int k = 0; k < VN; k++) sdg[warp * D + (v * 32 + lane) * VN + k] = dg[v][k];
    }
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += NTHR) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; w++) s += sdg[w * D + c];
    dgamma_part[(size_t)task * D + c] = s;
  }
  __syncthreads();
}

// dgamma[c] (=|+=) sum_b part[b, c], the partials taken in a fixed order: four interleaved running sums (b mod 4), so that four
// loads are in flight per thread instead of one, added at the end. Task = 256 columns. GT = gradient storage type.
template <class GT>
__device__ __forceinline__ void ln_dgamma_reduce_task(int task, GT* dgamma, const float* part, int nblk, int D, int accumulate) {
  const int c = task * NTHR + threadIdx.x;
  if (c < D) {
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    int b = 0;
    for (; b + 4 <= nblk; b += 4) {
#pragma unroll
      for (int q = 0; q < 4; q++) s[q] += part[(size_t)(b + q) * D + c];
    }
    for (; b < nblk; b++) s[b & 3] += part[(size_t)b * D + c];
    const float tot = (s[0] + s[1]) + (s[2] + s[3]);
    dgamma[c] = from_f<GT>(accumulate ? to_f(dgamma[c]) + tot : tot);
  }
}

// ---------------------------------------------------------------------------------------------- cross-entropy
// In place: logits[r,:] -> dlogits[r,:] = (softmax - onehot(target)) * inv_n;  loss[r] = logsumexp - logit[target].
// Pass 1 keeps the row in shared memory (as much as fits in `cache_bytes`), so pass 2 re-reads global memory only for the
// tail; the bf16 GPT-S row (100,608 B) fits entirely, i.e. the task moves the algorithmic minimum of 2 x row bytes.
// Task = CE_ROWS rows. Shared memory: 64 B scratch + cache_bytes.
template <class T>
__device__ __forceinline__ void ce_task(int task, T* logits, const int* targets, float* loss, int N, int V, float inv_n,
                                        unsigned char* smem, int cache_bytes) {
  constexpr int VN = (sizeof(T) == 2) ? 8 : 1;        // fp32 rows (tiny model) are not 16-byte aligned: scalar access
  constexpr float L2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
  float* red = reinterpret_cast<float*>(smem);
  T* cache = reinterpret_cast<T*>(smem + 64);
  const int t = threadIdx.x;
  const int nvec = V / VN;
  const int cvec = min(nvec, cache_bytes / (int)(VN * sizeof(T)));
  for (int rr = 0; rr < CE_ROWS; rr++) {
    const int r = task * CE_ROWS + rr;
    if (r >= N) break;
    T* row = logits + (size_t)r * V;
    const int tgt = targets[r];
    float m = -INFINITY, s = 0.f;
    for (int v = t; v < nvec; v += NTHR) {
      float f[VN];
      if constexpr (VN == 8) {
        const uint4 u = *reinterpret_cast<const uint4*>(row + (size_t)v * 8);
        if (v < cvec) *reinterpret_cast<uint4*>(cache + (size_t)v * 8) = u;
        unpack8(u, f);
      } else {
        f[0] = to_f(row[v]);
        if (v < cvec) cache[v] = row[v];
      }
      float cm = f[0];
#pragma unroll
      for (int k = 1; k < VN; k++) cm = fmaxf(cm, f[k]);
      cm *= L2E;
      if (cm > m) { s *= exp2f(m - cm); m = cm; }
#pragma unroll
      for (int k = 0; k < VN; k++) s += exp2f(fmaf(f[k], L2E, -m));
    }
    float lt = 0.f;
    if (t == 0) lt = to_f(row[tgt]);           // read before any thread overwrites the row (ordered by the syncs below)
    const float M = block_max(m, red);
    const float S = block_sum(s * exp2f(m - M), red);
    if (t == 0) loss[r] = M * LN2 + logf(S) - lt;
    const float invS = 1.f / S;
    for (int v = t; v < nvec; v += NTHR) {
      float f[VN];
      if constexpr (VN == 8) {
        const uint4 u = (v < cvec) ? *reinterpret_cast<const uint4*>(cache + (size_t)v * 8) : *reinterpret_cast<const uint4*>(row + (size_t)v * 8);
        unpack8(u, f);
      } else {
        f[0] = (v < cvec) ? to_f(cache[v]) : to_f(row[v]);
      }
#pragma unroll
      for (int k = 0; k < VN; k++) {
        float p = exp2f(fmaf(f[k], L2E, -M)) * invS;
        if (v * VN + k == tgt) p -= 1.f;
        f[k] = p * inv_n;
      }
      if constexpr (VN == 8) *reinterpret_cast<uint4*>(row + (size_t)v * 8) = pack8(f);
      else row[v] = from_f<T>(f[0]);
    }
    __syncthreads();   // cache and scratch are reused by the next row
  }
}

// The same task for bf16 rows that fit the cache entirely: the row is brought into shared memory by bulk copies (the copy
// engine streams it without occupying the threads or their registers; with the loop of 16-byte loads above a thread had one
// or two loads in flight and the phase ran at a third of the HBM rate), then both passes read shared memory. The arithmetic
// and its order are those of ce_task. `bar` is a block-private mbarrier, `uses` its running use count (advanced here).
__device__ __forceinline__ void ce_task_bulk(int task, bf16* logits, const int* targets, float* loss, int N, int V, float inv_n,
                                             unsigned char* smem, uint32_t bar, uint32_t& uses, const DevStatus* st) {
  constexpr float L2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
  float* red = reinterpret_cast<float*>(smem);
  bf16* cache = reinterpret_cast<bf16*>(smem + 64);
  const uint32_t cache_addr = smem_u32(cache);
  const int t = threadIdx.x;
  const int nvec = V / 8;
  const uint32_t row_bytes = (uint32_t)V * 2u;
  const uint32_t use0 = uses;
  uses += CE_ROWS;                                     // every thread, whatever happens below
  for (int rr = 0; rr < CE_ROWS; rr++) {
    const int r = task * CE_ROWS + rr;
    const uint32_t parity = (use0 + rr) & 1u;
    if (r >= N) { if (t == 0) mbar_arrive(bar); continue; }          // keep the barrier's phase count in step with `uses`
    bf16* row = logits + (size_t)r * V;
    if (t == 0) {
      fence_proxy_async();   // the row was written by a GEMM epilogue with ordinary stores; the cache was last read by ordinary loads
      mbar_expect_tx(bar, row_bytes);
      for (uint32_t off = 0; off < row_bytes; off += 32768u) {
        const uint32_t nb = row_bytes - off < 32768u ? row_bytes - off : 32768u;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(cache_addr + off), "l"(reinterpret_cast<const char*>(row) + off), "r"(nb), "r"(bar) : "memory");
      }
    }
    const int tgt = targets[r];
    bool ok = true;
    if (t == 0) {                                      // one thread polls; the block barrier below hands the result (and the data) to the rest
      ok = mbar_wait(bar, parity, st);
      if (!ok) { for (int spin = 0; spin < 100000 && !mbar_try(bar, parity); spin++) {} }   // leaving: give the copy a bounded chance to land
    }
    if (__syncthreads_or(!ok)) return;
    float m = -INFINITY, s = 0.f;
    for (int v = t; v < nvec; v += NTHR) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(cache + (size_t)v * 8), f);
      float cm = f[0];
#pragma unroll
      for (int k = 1; k < 8; k++) cm = fmaxf(cm, f[k]);
      cm *= L2E;
      if (cm > m) { s *= exp2f(m - cm); m = cm; }
#pragma unroll
      for (int k = 0; k < 8; k++) s += exp2f(fmaf(f[k], L2E, -m));
    }
    float lt = 0.f;
    if (t == 0) lt = to_f(cache[tgt]);
    const float M = block_max(m, red);
    const float S = block_sum(s * exp2f(m - M), red);
    if (t == 0) loss[r] = M * LN2 + logf(S) - lt;
    const float invS = 1.f / S;
    for (int v = t; v < nvec; v += NTHR) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(cache + (size_t)v * 8), f);
#pragma unroll
      for (int k = 0; k < 8; k++) {
        float p = exp2f(fmaf(f[k], L2E, -M)) * invS;
        if (v * 8 + k == tgt) p -= 1.f;
        f[k] = p * inv_n;
      }
      *reinterpret_cast<uint4*>(row + (size_t)v * 8) = pack8(f);
    }
    __syncthreads();   // cache and scratch are reused by the next row
  }
}

// Cross-entropy behind an LM-head GEMM whose epilogue left softmax partials (GE_LSE): per row and 128-column tile the maximum m_t
// of x * log2(e) over the stored values and s_t = sum 2^(x * log2(e) - m_t). The row's maximum and sum follow from the tiles_n
// partials (a few KB) without touching the logits, so the logits are read ONCE and rewritten in the same pass:
//   M = max_t m_t,  S = sum_t s_t * 2^(m_t - M)  (fixed order),  loss = M * ln2 + ln S - logit[target],
//   dlogit = (2^(x * log2(e) - M) / S - onehot) * inv_n.
// The task's rows move through shared memory as one stream of chunks staged by the copy engine, four chunks (96 KB) in flight
// across row boundaries; nothing waits for a whole row. `bar_lo`, `bar_hi` = two pairs of block-private mbarriers (count 1), `chunks` = running
// count of chunks this block has staged (advanced identically by every thread). V must be a multiple of 8.
constexpr int CE_CHUNK = 12288, CE_STAGES = 4;            // elements per chunk (24 KB of bf16)
static __device__ __noinline__ void ce_task_stream(int task, bf16* logits, const int* targets, float* loss, const float2* part, int tiles_n,
                                               int N, int V, float inv_n, unsigned char* smem, uint32_t bar_lo, uint32_t bar_hi, uint32_t& chunks,
                                               const DevStatus* st) {
  auto sbar = [&](uint32_t sg) { return sg < 2 ? bar_lo + 8u * sg : bar_hi + 8u * (sg - 2); };   // the four barriers sit in two free pairs of the control area
  constexpr float L2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;
  float* rowMS = reinterpret_cast<float*>(smem + CE_STAGES * CE_CHUNK * 2);        // [CE_ROWS][2] behind the stages: M and 1/S of the task's rows
  const int t = threadIdx.x;
  const int r0 = task * CE_ROWS, nrows = min(CE_ROWS, N - r0);
  const int cpr = (V + CE_CHUNK - 1) / CE_CHUNK;                                   // chunks per row
  const int total = nrows > 0 ? nrows * cpr : 0;
  const uint32_t u0 = chunks;
  chunks += (uint32_t)total;                                                       // every thread, whatever happens below
  const uint32_t sbase = smem_u32(smem);
  auto issue = [&](int k) {                                                        // thread 0: chunk k of this task into stage (u0 + k) % 4
    const uint32_t u = u0 + (uint32_t)k, sg = u % CE_STAGES, b = sbar(sg);
    const int rr = k / cpr, c0 = (k % cpr) * CE_CHUNK;
    const uint32_t bytes = (uint32_t)min(CE_CHUNK, V - c0) * 2u;
    mbar_expect_tx(b, bytes);
    bulk_g2s(sbase + sg * (CE_CHUNK * 2), logits + (size_t)(r0 + rr) * V + c0, bytes, b);
  };
  if (t == 0 && total > 0) {
    fence_proxy_async();     // the rows were written by a GEMM epilogue with ordinary stores; the stages were last read by ordinary loads
    for (int k = 0; k < CE_STAGES && k < total; k++) issue(k);
  }
  // row statistics from the partials while the first chunks travel: one warp per row, lanes over the tiles, fixed reduction order
  {
    const int warp = t >> 5, lane = t & 31;
    if (warp < nrows) {
      const int rr = warp;
      const float2* pr = part + (size_t)(r0 + rr) * tiles_n;
      float m = -INFINITY;
      for (int i = lane; i < tiles_n; i += 32) m = fmaxf(m, pr[i].x);
      const float M = warp_max(m);
      float sm = 0.f;
      for (int i = lane; i < tiles_n; i += 32) { const float2 v = pr[i]; sm += v.y * exp2f(v.x - M); }
      const float S = warp_sum(sm);
      if (lane == 0) {
        rowMS[2 * rr] = M; rowMS[2 * rr + 1] = 1.f / S;
        loss[r0 + rr] = M * LN2 + logf(S) - to_f(logits[(size_t)(r0 + rr) * V + targets[r0 + rr]]);   // read before the row's chunks are rewritten (ordered by the barrier below)
      }
    }
  }
  __syncthreads();
  for (int k = 0; k < total; k++) {
    const uint32_t u = u0 + (uint32_t)k, sg = u % CE_STAGES;
    const bool ok = mbar_wait(sbar(sg), (u / CE_STAGES) & 1u, st);
    if (ok) {
      const int rr = k / cpr, c0 = (k % cpr) * CE_CHUNK, len = min(CE_CHUNK, V - c0);
      const float M = rowMS[2 * rr], scale = rowMS[2 * rr + 1] * inv_n;             // p * inv_n = 2^(x log2e - M) * (inv_n / S)
      const int tgt = targets[r0 + rr] - c0;                                       // position of the target inside this chunk, if it is there
      const bf16* src = reinterpret_cast<const bf16*>(smem + sg * (CE_CHUNK * 2));
      bf16* dst = logits + (size_t)(r0 + rr) * V + c0;
      for (int v = t * 8; v < len; v += NTHR * 8) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(src + v), f);
#pragma unroll
        for (int i = 0; i < 8; i++) f[i] = ex2_approx(fmaf(f[i], L2E, -M)) * scale;
        if ((unsigned)(tgt - v) < 8u) {                                             // the one-hot term: (p - 1) * inv_n (no dynamic register index)
#pragma unroll
          for (int i = 0; i < 8; i++) if (tgt - v == i) f[i] -= inv_n;
        }
        *reinterpret_cast<uint4*>(dst + v) = pack8(f);
      }
    }
    if (__syncthreads_or(!ok)) {                        // giving up (abort or deadline): let the copies still in flight land, then leave
      if (t == 0)
        for (int kk = k; kk < total && kk < k + CE_STAGES; kk++) {
          const uint32_t uu = u0 + (uint32_t)kk;
          for (int spin = 0; spin < 100000 && !mbar_try(sbar(uu % CE_STAGES), (uu / CE_STAGES) & 1u); spin++) {}
        }
      __syncthreads();
      return;
    }
    if (t == 0 && k + CE_STAGES < total) { fence_proxy_async(); issue(k + CE_STAGES); }
  }
}

// mean_loss[0] = (sum_r loss[r]) / N, fixed order. One task.
__device__ __forceinline__ float ce_mean_task(float* mean_loss, const float* loss, int N, unsigned char* smem) {
  float s = 0.f;
  for (int i = threadIdx.x; i < N; i += NTHR) s += loss[i];
  s = block_sum(s, reinterpret_cast<float*>(smem));
  const float m = s / (float)N;
  if (threadIdx.x == 0) mean_loss[0] = m;
  return m;
}

// ---------------------------------------------------------------------------------------------- embedding backward
__host__ __device__ constexpr size_t embed_bwd_wte_smem_bytes(int N) { return 1024 + 5 * (size_t)N; }

// dwte[v,:] (=|+=) sum over tokens n with tok[n] == v of dx0[n,:], added in increasing n (the reference's order,
// llm/elementwise/ew_loss.cuh:101-177, so that the sum does not depend on the schedule). Task = 128 vocabulary rows.
//   1. Each warp looks at its own contiguous eighth of the token positions, 32 at a time: ballots count its matches (and a shared
//      counter per row says how many each row has; most rows of a chunk have none), the eight warp counts give it its place in an
//      ORDERED list of (position, row) pairs, and a second look at the same positions fills the list.
//   2. A warp owns rows w, w + 8, ...; for a row with pairs it walks the list 32 entries at a time (ballot of "this entry is
//      mine"), adding the dx0 rows in list order into registers (a lane holds vectors lane, lane + 32, ... of the row).
// Without `accumulate` every row of the chunk is written (zeros where the token is absent), so the gradient buffer needs no
// clearing between steps. Shared memory: 8 warp counts + 128 row counts, then int list[N], then one byte per list entry.
template <class T, int D, class GT>
__device__ __noinline__ void embed_bwd_wte_task(int task, GT* dwte, const T* dx0, const int* tok, int N, int V, int accumulate,
                                                unsigned char* smem) {
  using R = RowRegs<T, D>;
  constexpr int VN = R::VN, NV = R::NV;
  int* wcnt = reinterpret_cast<int*>(smem);            // [8]
  int* rowcnt = wcnt + 8;                              // [EMB_VCHUNK]
  int* list = reinterpret_cast<int*>(smem + 1024);     // [N] matching positions, increasing
  unsigned char* rowof = smem + 1024 + 4 * (size_t)N;  // [N] row within the chunk of each list entry
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31, lo = task * EMB_VCHUNK;
  if (t < EMB_VCHUNK) rowcnt[t] = 0;
  __syncthreads();
  // warp w owns positions [w * per, (w + 1) * per): its matches follow those of the warps before it, in position order
  const int per = ((N + NTHR - 1) / NTHR) * 32, p0 = warp * per, p1 = min(N, p0 + per);
  int mine_cnt = 0;
#pragma unroll 4
  for (int n = p0 + lane; n < p0 + per; n += 32) {
    const int v = n < p1 ? tok[n] - lo : -1;
    const bool hit = (unsigned)v < (unsigned)EMB_VCHUNK;
    mine_cnt += __popc(__ballot_sync(0xffffffffu, hit));
    if (hit) atomicAdd(&rowcnt[v], 1);
  }
  if (lane == 0) wcnt[warp] = mine_cnt;
  __syncthreads();
  int slot = 0, total = 0;
#pragma unroll
  for (int w = 0; w < NTHR / 32; w++) { const int c = wcnt[w]; total += c; if (w < warp) slot += c; }
  for (int n = p0 + lane; n < p0 + per && mine_cnt > 0; n += 32) {      // second look at the same positions (now in L1): place the matches
    const int v = n < p1 ? tok[n] - lo : -1;
    const bool hit = (unsigned)v < (unsigned)EMB_VCHUNK;
    const unsigned b = __ballot_sync(0xffffffffu, hit);
    if (hit) { const int at = slot + __popc(b & ((1u << lane) - 1u)); list[at] = n; rowof[at] = (unsigned char)v; }
    slot += __popc(b);
  }
  __syncthreads();
  for (int r = warp; r < EMB_VCHUNK; r += NTHR / 32) {
    if (lo + r >= V) break;
    GT* dst = dwte + (size_t)(lo + r) * D;
    const int mine = rowcnt[r];
    if (mine == 0 && accumulate) continue;
    float acc[NV][VN];
#pragma unroll
    for (int v = 0; v < NV; v++) {
      const int vi = v * 32 + lane;
#pragma unroll
      for (int k = 0; k < VN; k++) acc[v][k] = (accumulate && vi < R::VPR) ? to_f(dst[vi * VN + k]) : 0.f;
    }
    int seen = 0;
    for (int k0 = 0; k0 < total && seen < mine; k0 += 32) {
      const int k = k0 + lane;
      unsigned m = __ballot_sync(0xffffffffu, k < total && rowof[k] == r);
      seen += __popc(m);
      while (m) {
        const T* src = dx0 + (size_t)list[k0 + __ffs(m) - 1] * D;
        m &= m - 1;
#pragma unroll
        for (int v = 0; v < NV; v++) {
          const int vi = v * 32 + lane;
          if (vi < R::VPR) {
            float f[VN]; ldv(src + vi * VN, f);
#pragma unroll
            for (int kk = 0; kk < VN; kk++) acc[v][kk] += f[kk];
          }
        }
      }
    }
#pragma unroll
    for (int v = 0; v < NV; v++) {
      const int vi = v * 32 + lane;
      if (vi < R::VPR) {
#pragma unroll
        for (int k = 0; k < VN; k += 4) st4(dst + vi * VN + k, &acc[v][k]);
      }
    }
  }
  __syncthreads();
}

// dwpe32[p,:] (=) sum_b dx0[b*Tctx + p,:], b increasing. Task = 4 positions.
template <class T, class GT>
__device__ __forceinline__ void embed_bwd_wpe_task(int task, GT* dwpe32, const T* dx0, int N, int Tctx, int D) {
  for (int pp = 0; pp < WPE_ROWS; pp++) {
    const int p = task * WPE_ROWS + pp;
    if (p >= Tctx) break;
    for (int c = threadIdx.x; c < D; c += NTHR) {
      float s = 0.f;
      for (int n = p; n < N; n += Tctx) s += to_f(dx0[(size_t)n * D + c]);
      dwpe32[(size_t)p * D + c] = from_f<GT>(s);
    }
  }
}

// ---------------------------------------------------------------------------------------------- AdamW
struct AdamHP { float lr, beta1, beta2, eps, weight_decay, grad_scale; int step; };   // step is 1-based

__device__ __forceinline__ float lr_at(const AdamConst& h, int s) {
  if (h.constant_lr) return h.lr_max;
  if (s < h.warmup) return h.lr_max * (float)(s + 1) / (float)h.warmup;
  const double p = (double)(s - h.warmup) / (double)(h.sched_steps - h.warmup);
  const double q = p < 1.0 ? p : 1.0;
  return (float)(h.lr_min + 0.5 * (h.lr_max - h.lr_min) * (1.0 + cos(3.14159265358979323846 * q)));
}
__device__ __forceinline__ AdamHP adam_hp(const AdamConst& h, int step) {
  AdamHP hp; hp.lr = lr_at(h, step); hp.beta1 = h.beta1; hp.beta2 = h.beta2; hp.eps = h.eps; hp.weight_decay = h.wd;
  hp.grad_scale = h.grad_scale; hp.step = step + 1; return hp;
}

// torch.optim.AdamW (non-fused, non-amsgrad) operation order on fp32 master weights, as the reference keeps it
// (llm/elementwise/ew_adamw.cuh:20-67):
//   p *= 1 - lr*wd (unless the element lies in a no-decay range) ; m += (g - m)(1 - b1) ; v = fma(v, b2, (1 - b2) g^2) ;
//   p -= lr/(1 - b1^t) * m / (sqrt(v)/sqrt(1 - b2^t) + eps)          (bias corrections in double)
// then the working copy Wact (type T) that forward, backward and the decoder read is refreshed. The gradient is read as GT
// (fp32 single-GPU buffer, or the all-reduced bf16 bucket) and multiplied by grad_scale (1/world size).
// nodecay: sorted disjoint [start,end) element ranges relative to W. Task = 65,536 elements; n and ranges multiples of 4.
struct AdamMath {                     // the per-task constants and the four-element update shared by both task bodies
  float step_size, inv_sqrt_bc2, decay_mul, one_minus_b1, one_minus_b2, b2, eps, gscale;
  const int2* nd; int n_nd, first_nd; bool any_nd;
  __device__ __forceinline__ void init(const AdamHP& hp, const int2* nodecay, int n_nodecay, size_t chunk_begin, size_t chunk_end) {
    const double bc1 = 1.0 - pow((double)hp.beta1, (double)hp.step), bc2 = 1.0 - pow((double)hp.beta2, (double)hp.step);
    step_size = (float)((double)hp.lr / bc1);
    inv_sqrt_bc2 = (float)(1.0 / sqrt(bc2));
    decay_mul = 1.f - hp.lr * hp.weight_decay;
    one_minus_b1 = 1.f - hp.beta1; one_minus_b2 = 1.f - hp.beta2; b2 = hp.beta2; eps = hp.eps; gscale = hp.grad_scale;
    nd = nodecay; n_nd = n_nodecay;
    int lo = 0, hi = n_nodecay;       // first range whose end lies beyond the chunk start
    while (lo < hi) { const int mid = (lo + hi) >> 1; if ((size_t)nodecay[mid].y <= chunk_begin) lo = mid + 1; else hi = mid; }
    first_nd = lo;
    any_nd = lo < n_nodecay && (size_t)nodecay[lo].x < chunk_end;
  }
  __device__ __forceinline__ bool decays(size_t idx) const {
    if (!any_nd) return true;
    int ri = first_nd;
    while (ri < n_nd && (size_t)nd[ri].y <= idx) ri++;
    return !(ri < n_nd && idx >= (size_t)nd[ri].x);
  }
  __device__ __forceinline__ void update4(size_t i, float* w, const float* g, float* m, float* v) const {
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const float gg = g[k] * gscale;
      const float p = decays(i + k) ? w[k] * decay_mul : w[k];
      m[k] = m[k] + (gg - m[k]) * one_minus_b1;
      v[k] = fmaf(v[k], b2, one_minus_b2 * gg * gg);
      w[k] = p - step_size * (m[k] / (sqrtf(v[k]) * inv_sqrt_bc2 + eps));
    }
  }
};
// elements [begin, end) with loads issued by the threads themselves (the fp32 preset, and the ragged end of a staged task)
template <class T, class GT>
__device__ __forceinline__ void adamw_span_direct(const AdamMath& A, size_t begin, size_t end, float* W, const GT* G, float* M, float* Vv, T* Wact) {
#pragma unroll 4
  for (size_t i = begin + (size_t)threadIdx.x * 4; i < end; i += NTHR * 4) {
    float w[4], g[4], m[4], v[4];
    ld4(W + i, w); ld4(G + i, g); ld4(M + i, m); ld4(Vv + i, v);
    A.update4(i, w, g, m, v);
    st4(W + i, w); st4(M + i, m); st4(Vv + i, v); st4(Wact + i, w);
  }
}
template <class T, class GT>
__device__ __forceinline__ void adamw_task(int task, float* W, const GT* G, float* M, float* Vv, T* Wact, size_t n, AdamHP hp,
                                           const int2* nodecay, int n_nodecay) {
  const size_t cs = (size_t)task * OPT_CHUNK;
  if (cs >= n) return;
  const size_t ce = cs + OPT_CHUNK < n ? cs + OPT_CHUNK : n;
  AdamMath A; A.init(hp, nodecay, n_nodecay, cs, ce);
  adamw_span_direct<T, GT>(A, cs, ce, W, G, M, Vv, Wact);
}

// The same update with the inputs staged through shared memory by the copy engine. A block has 8 warps and each thread can keep
// only a few 16-byte loads in flight, so the loop above runs at what 256 threads can request, not at what HBM can deliver
// (measured: 0.71 of the copy bandwidth with every block of the GPU running it, 0.90 staged). One thread queues bulk copies
// (cp.async.bulk, completion counted on an mbarrier) of W, M, V and G for tiles of 2,048 elements, three tiles (96 KB) ahead
// of the arithmetic; the threads read their operands from shared memory and write results straight to global memory.
// `bar0` = three block-private mbarriers (count 1), `tiles` = running count of tiles this block has staged since it started
// (advanced identically by every thread). The ragged end of a range (fewer than 2,048 elements) goes through the direct loop.
constexpr int ADAM_TILE = 2048, ADAM_STAGES = 3, ADAM_STAGE_BYTES = 32768;
template <class T, class GT>
__device__ __noinline__ void adamw_task_bulk(int task, float* W, const GT* G, float* M, float* Vv, T* Wact, size_t n, AdamHP hp,
                                                const int2* nodecay, int n_nodecay, unsigned char* smem, uint32_t bar0, uint32_t& tiles,
                                                const DevStatus* st) {
  const size_t cs = (size_t)task * OPT_CHUNK;
  if (cs >= n) return;
  const size_t ce = cs + OPT_CHUNK < n ? cs + OPT_CHUNK : n;
  AdamMath A; A.init(hp, nodecay, n_nodecay, cs, ce);
  const int tid = threadIdx.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(M) | reinterpret_cast<uintptr_t>(Vv) | reinterpret_cast<uintptr_t>(G)) & 15) == 0;
  const int nfull = aligned ? (int)((ce - cs) / ADAM_TILE) : 0;
  const uint32_t u0 = tiles;
  tiles += (uint32_t)nfull;                             // every thread, whatever happens below
  const uint32_t sbase = smem_u32(smem);
  auto issue = [&](int k) {                            // thread 0: tile k of this task into stage (u0 + k) % 3
    const uint32_t u = u0 + (uint32_t)k, s = u % ADAM_STAGES, b = bar0 + 8u * s, dst = sbase + s * ADAM_STAGE_BYTES;
    const size_t i0 = cs + (size_t)k * ADAM_TILE;
    mbar_expect_tx(b, 3u * ADAM_TILE * 4u + (uint32_t)(ADAM_TILE * sizeof(GT)));
    bulk_g2s(dst, W + i0, ADAM_TILE * 4, b); bulk_g2s(dst + 8192, M + i0, ADAM_TILE * 4, b);
    bulk_g2s(dst + 16384, Vv + i0, ADAM_TILE * 4, b); bulk_g2s(dst + 24576, G + i0, (uint32_t)(ADAM_TILE * sizeof(GT)), b);
  };
  if (tid == 0 && nfull > 0) {
    fence_proxy_async();     // gradients and the previous step's W/M/V were written with ordinary stores; the stages were last read by ordinary loads
    for (int k = 0; k < ADAM_STAGES && k < nfull; k++) issue(k);
  }
  for (int k = 0; k < nfull; k++) {
    const uint32_t u = u0 + (uint32_t)k, s = u % ADAM_STAGES;
    const bool ok = mbar_wait(bar0 + 8u * s, (u / ADAM_STAGES) & 1u, st);
    if (ok) {
      const unsigned char* sp = smem + s * ADAM_STAGE_BYTES;
      const size_t i0 = cs + (size_t)k * ADAM_TILE;
#pragma unroll
      for (int q = 0; q < ADAM_TILE / (NTHR * 4); q++) {
        const int e = q * NTHR * 4 + tid * 4;             // a warp touches 512 contiguous bytes of each array: no bank conflicts
        float w[4], g[4], m[4], v[4];
        ld4(reinterpret_cast<const float*>(sp) + e, w); ld4(reinterpret_cast<const float*>(sp + 8192) + e, m);
        ld4(reinterpret_cast<const float*>(sp + 16384) + e, v); ld4(reinterpret_cast<const GT*>(sp + 24576) + e, g);
        A.update4(i0 + e, w, g, m, v);
        st4(W + i0 + e, w); st4(M + i0 + e, m); st4(Vv + i0 + e, v); st4(Wact + i0 + e, w);
      }
    }
    if (__syncthreads_or(!ok)) {                        // giving up (abort or deadline): let the copies still in flight land, then leave
      if (tid == 0)
        for (int kk = k; kk < nfull && kk < k + ADAM_STAGES; kk++) {
          const uint32_t uu = u0 + (uint32_t)kk;
          for (int spin = 0; spin < 100000 && !mbar_try(bar0 + 8u * (uu % ADAM_STAGES), (uu / ADAM_STAGES) & 1u); spin++) {}
        }
      __syncthreads();
      return;
    }
    if (tid == 0 && k + ADAM_STAGES < nfull) { fence_proxy_async(); issue(k + ADAM_STAGES); }
  }
  adamw_span_direct<T, GT>(A, cs + (size_t)nfull * ADAM_TILE, ce, W, G, M, Vv, Wact);
}

// out[i] = T(part0[i] + part1[i] + ...) in index order: the reduce of a split-K GEMM. Task = 16,384 elements (n % 8 == 0).
template <class T>
__device__ __forceinline__ void sumcast_task(int task, T* out, void* const* parts, int nparts, size_t n) {
  const size_t s0 = (size_t)task * SUM_CHUNK, e0 = s0 + SUM_CHUNK < n ? s0 + SUM_CHUNK : n;
  for (size_t i = s0 + (size_t)threadIdx.x * 8; i < e0; i += NTHR * 8) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; k++) acc[k] = 0.f;
    for (int p = 0; p < nparts; p++) {
      const float* src = reinterpret_cast<const float*>(parts[p]) + i;
      const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w; acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
#pragma unroll
    for (int k = 0; k < 8; k++) out[i + k] = from_f<T>(acc[k]);
  }
}

// tok_in / tok_tgt for sequence `seq` of step `step`: window start from the table, or a counter-based hash of the seed.
__device__ __forceinline__ void data_task(int seq, int step, const uint32_t* data, u64 ntok, const uint32_t* starts, int nstarts,
                                          u64 seed, int* tok_in, int* tok_tgt, int Tctx, int B) {
  u64 st;
  if (starts) st = starts[(size_t)(step % nstarts) * B + seq];
  else st = splitmix64(seed ^ ((u64)step * B + seq)) % (ntok - Tctx - 1);
  for (int t = threadIdx.x; t < Tctx; t += NTHR) {
    tok_in[seq * Tctx + t] = (int)data[st + t];
    tok_tgt[seq * Tctx + t] = (int)data[st + t + 1];
  }
}

}  // namespace ew
}  // namespace ofa
