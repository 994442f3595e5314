// bf16 tensor-core GEMM task for sm_100a: TMA -> swizzled shared memory -> tcgen05.mma -> TMEM -> epilogue.
//
// Task contract (replaces the reference's `tg::tile<LAYOUT,EPI>` = gemm::sm100::tile_tc,
// llm/b200/gemm_tcgen05/gemm_sm100.cuh:174-289, with the layouts/epilogues of llm/gemm/gemm.cuh:18-50):
//   one task = a STRIP of `nsub` consecutive 128 x BN tiles of C that share their 128 rows; all 256 threads call
//   gemm_tc_task() together. BN is 128 by default; 256 is an opt-in per GEMM. Differences in design from the reference tile:
//     * two tile widths. With every SM busy a 64-deep K step of a 128x128 tile takes 0.66 us per block (~14 TB/s of operand
//       reads GPU-wide); a 128x256 tile moves 48 KB instead of 64 KB per 128x256x64 of work but fits only two stages per
//       block, and measured slower on all model shapes except lm_head dW: the loop is bound by bytes in flight;
//     * the mbarriers and the 256 TMEM columns of a block live for the whole kernel; phase parities are derived from running
//       counters kept in `GemmPipe` (one set of barriers and counters per tile width, because the widths use different
//       pipeline depths), so nothing is re-initialised or invalidated between tiles or tasks;
//     * inside a strip the TMA producer (warp 0) and the MMA issuer (warp 1) run ahead of the epilogue; with BN = 128 the
//       accumulator is double-buffered in TMEM (2 x 128 columns) and drained by warps 4..7 while the next tile's MMAs are in
//       flight; with BN = 256 one accumulator fills the block's TMEM and the SM's other resident block provides the overlap;
//     * the epilogue never touches the pipeline buffers: each epilogue warp transposes 32x32 fp32 blocks through its own
//       4 KB staging area (XOR-swizzled, conflict-free) and then moves whole 64/128-byte row segments to global memory;
//       epilogues that read `aux` fetch their row segments before waiting for the accumulator;
//     * every wait is bounded and aborts the grid cleanly on expiry.
//   K order is fixed (k ascending, one accumulator) => results are deterministic and independent of the schedule and of BN.
//
// Operand staging (SWIZZLE_128B everywhere; one pipeline stage = 64 values of K: 16 KB of A + BN x 128 B of B):
//   K-major operand  X[rows][K]  (A of NN/NT, B of NT): TMA boxes {64 k, 128 rows} -> 128 rows x 128 B each; UMMA descriptor
//     SBO = 1024 B (8 rows), a step of 16 in K advances the start address by 32 B.
//   MN-major operand X[K][cols]  (B of NN/TN, A of TN): TMA boxes {64 cols, 64 k}, 8 KB apart -> per box 64 k-rows x
//     128 B; UMMA descriptor LBO = 8192 B (between 64-wide column groups), SBO = 1024 B (8 k-rows), a step of 16 in K
//     advances the start address by 2048 B.
#pragma once
#include "common.cuh"
#include "task_api.h"

namespace ofa {
namespace gemm_tc {

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;                 // 16 KB
constexpr int PIPE_BYTES = 96 * 1024;                // 3 stages x 32 KB (BN 128) or 2 stages x 48 KB (BN 256)
constexpr int EPI_WARPS = 4;                         // warps 4..7
constexpr int STAGING_BYTES = EPI_WARPS * 32 * 32 * 4;   // 16 KB
constexpr int BAR_OFFSET = PIPE_BYTES + STAGING_BYTES;   // control area: barriers, TMEM slot, scheduler words
constexpr int BAR_BYTES = CTRL_BYTES;
constexpr int SMEM_BYTES = BAR_OFFSET + BAR_BYTES;   // 115,712 B: two blocks per SM use the whole 228 KB (1 KB per block is reserved by the system)
constexpr int TMEM_COLS = 256;

template <int BN> struct Cfg {
  static constexpr int W = BN == 128 ? 0 : 1;                    // which barrier set / counter set
  static constexpr int STAGES = BN == 128 ? 3 : 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int NBUF = BN == 128 ? 2 : 1;                  // accumulators in TMEM
  static constexpr int BAR0 = BN == 128 ? 0 : 176;                // byte offset of this width's barriers in the control area
  static_assert(STAGES * STAGE_BYTES <= PIPE_BYTES, "pipeline does not fit");
};
// control area (1 KB at smem + BAR_OFFSET = the last 1,024 bytes of dynamic shared memory):
//   [  0, 80) BN128: full[3] empty[3] accf[2] acce[2]     [ 80, 84) TMEM base slot     [ 96,104) serving fill barrier   [104,112) training bulk-copy barrier
//   [112,128) and [160,176) streamed cross-entropy stage barriers [4]
//   [128,160) scheduler hand-off words                      [176,224) BN256: full[2] empty[2] accf[1] acce[1]      [224,248) AdamW stage barriers [3]
//   [256,512) and [512,768) two slots for phase descriptors: the one being worked on and the next phase's, fetched ahead
//   [768,832) scheduling record (ticket range + dependencies) of the phase the scheduler thread looks at next
template <int BN> __device__ __forceinline__ uint32_t bar_full(uint32_t base, int s) { return base + BAR_OFFSET + Cfg<BN>::BAR0 + 8u * s; }
template <int BN> __device__ __forceinline__ uint32_t bar_empty(uint32_t base, int s) { return base + BAR_OFFSET + Cfg<BN>::BAR0 + 8u * (Cfg<BN>::STAGES + s); }
template <int BN> __device__ __forceinline__ uint32_t bar_accf(uint32_t base, int b) { return base + BAR_OFFSET + Cfg<BN>::BAR0 + 8u * (2 * Cfg<BN>::STAGES + b); }
template <int BN> __device__ __forceinline__ uint32_t bar_acce(uint32_t base, int b) { return base + BAR_OFFSET + Cfg<BN>::BAR0 + 8u * (2 * Cfg<BN>::STAGES + Cfg<BN>::NBUF + b); }
constexpr int TMEM_SLOT_OFFSET = BAR_OFFSET + 80;

// Per-thread running counters, one set per tile width; every thread advances them identically at the end of a task.
struct GemmPipe {
  uint32_t stage_count[2];   // pipeline stages produced/consumed since block start
  uint32_t tile_count[2];    // accumulator tiles since block start
  uint32_t tmem_base;
};

template <int BN> __device__ __forceinline__ void init_bars(uint32_t base) {
  for (int s = 0; s < Cfg<BN>::STAGES; s++) { mbar_init(bar_full<BN>(base, s), 1); mbar_init(bar_empty<BN>(base, s), 1); }
  for (int b = 0; b < Cfg<BN>::NBUF; b++) { mbar_init(bar_accf<BN>(base, b), 1); mbar_init(bar_acce<BN>(base, b), EPI_WARPS); }
}
// Once per block, before its first GEMM task. All 256 threads. Returns false (and aborts) if shared memory is misaligned.
__device__ __forceinline__ bool block_init(GemmPipe& gp, unsigned char* smem, DevStatus* st) {
  const uint32_t base = smem_u32(smem);
  gp.stage_count[0] = gp.stage_count[1] = 0; gp.tile_count[0] = gp.tile_count[1] = 0; gp.tmem_base = 0;
  const bool ok = (base & 1023u) == 0;
  if (!ok) { if (threadIdx.x == 0) raise_abort(st, ST_SMEM_MISALIGNED, -1, -1, (int)base); }
  if (threadIdx.x == 0) { init_bars<128>(base); init_bars<256>(base); mbar_fence_init(); }
  if (threadIdx.x < 32) tmem_alloc(base + TMEM_SLOT_OFFSET, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  gp.tmem_base = *reinterpret_cast<volatile uint32_t*>(smem + TMEM_SLOT_OFFSET);
  return ok;
}
// Once per block before it exits. All 256 threads. TMA copies still in flight when a task gives up are waited for
// (bounded) by the producer inside that task; here an aborting block only adds a short fixed delay before freeing TMEM.
__device__ __forceinline__ void block_exit(GemmPipe& gp, unsigned char* smem, DevStatus* st) {
  (void)smem;
  if (aborted(st)) __nanosleep(20000);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x < 32) tmem_dealloc(gp.tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------- epilogue math
// The epilogues that meet their second operand in fp32 before the one rounding (and the fp32 result): eight consecutive
// columns of one row, after the fp32 transpose. Everything else is stored from the bf16-staged pass of the task itself.
template <int EPI>
__device__ __forceinline__ void epi_store8(const GemmArgs& g, size_t row, int col, const float* acc, uint4 auxv) {
  static_assert(EPI == GE_F32 || EPI == GE_RES || EPI == GE_DGELU, "bf16 results without a second fp32 operand take the staged pass");
  if constexpr (EPI == GE_F32) {
    float* dst = reinterpret_cast<float*>(g.C) + row * g.ldc + col;
    float4 v0 = make_float4(acc[0], acc[1], acc[2], acc[3]), v1 = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if (g.accumulate) {
      const float4 o0 = *reinterpret_cast<const float4*>(dst), o1 = *reinterpret_cast<const float4*>(dst + 4);
      v0.x += o0.x; v0.y += o0.y; v0.z += o0.z; v0.w += o0.w; v1.x += o1.x; v1.y += o1.y; v1.z += o1.z; v1.w += o1.w;
    }
    *reinterpret_cast<float4*>(dst) = v0; *reinterpret_cast<float4*>(dst + 4) = v1;
  } else {
    float v[8], a8[8];
    unpack8(auxv, a8);
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = EPI == GE_RES ? acc[i] + a8[i] : acc[i] * gelu_bwd<true>(a8[i]);
    *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(g.C) + row * g.ldc + col) = pack8(v);
  }
}

// ---------------------------------------------------------------------------------------------- the task
// task index -> (tile_m, first tile_n): consecutive tasks walk down M first so that neighbouring blocks share the B strip.
template <int LAYOUT, int EPI, int BN>
__device__ __forceinline__ void gemm_tc_task(const GemmArgs& g, int tiles_m, int task, unsigned char* smem, GemmPipe& gp,
                                             DevStatus* st, int phase_id, const EarlyTicket& et, int nfast) {
  using CF = Cfg<BN>;
  constexpr bool A_MN = (LAYOUT == GL_TN), B_MN = (LAYOUT != GL_NT);
  constexpr bool HAS_AUX_IN = (EPI == GE_RES || EPI == GE_DGELU || EPI == GE_DR);
  constexpr bool BF16_STAGED = (EPI == GE_STORE || EPI == GE_GELU || EPI == GE_LSE || EPI == GE_DR);   // epilogues whose stored value is the rounded accumulator
  constexpr uint32_t IDESC = umma_idesc(A_MN, B_MN, BM, BN);
  constexpr int STAGES = CF::STAGES, W = CF::W;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t base = smem_u32(smem);
  const int KT = g.K / BK;
  const int tiles_n = g.N / BN;
  // nfast: consecutive tasks walk along N first, so the tasks that stream the same rows of a large A run side by side and the
  // second and third reader find them in L2 (the LM head's weight gradient); otherwise down M first, sharing the B strip
  const int nstrips = (tiles_n + g.nsub - 1) / g.nsub;
  const int tm = nfast ? task / nstrips : task % tiles_m, strip = nfast ? task % nstrips : task / tiles_m;
  const int tn0 = strip * g.nsub;
  const int nt = min(g.nsub, tiles_n - tn0);
  const int m0 = tm * BM;

  if (warp == 0) {
    if (lane == 0) {                                                           // ---- TMA producer
      fence_proxy_async();     // operands were written with ordinary stores by earlier phases (possibly other SMs)
      uint32_t sc = gp.stage_count[W];
      bool ok = true;
      for (int t = 0; t < nt && ok; t++) {
        const int n0 = (tn0 + t) * BN;
        for (int kt = 0; kt < KT; kt++, sc++) {
          const int s = sc % STAGES; const uint32_t use = sc / STAGES;
          const uint32_t full = bar_full<BN>(base, s);
          if (!mbar_wait(bar_empty<BN>(base, s), (use & 1) ^ 1, st)) { if (!aborted(st)) raise_abort(st, ST_MBAR_EMPTY_TIMEOUT, phase_id, task, kt); ok = false; break; }
          mbar_expect_tx(full, CF::STAGE_BYTES);
          const uint32_t sA = base + s * CF::STAGE_BYTES, sB = sA + A_BYTES;
          const int k0 = kt * BK;
          if (!A_MN) tma_load_2d(sA, g.tmA, full, k0, m0);
          else { tma_load_2d(sA, g.tmA, full, m0, k0); tma_load_2d(sA + 8192, g.tmA, full, m0 + 64, k0); }
          if (!B_MN) {
#pragma unroll
            for (int h = 0; h < BN / 128; h++) tma_load_2d(sB + h * 16384, g.tmB, full, k0, n0 + h * 128);
          } else {
#pragma unroll
            for (int h = 0; h < BN / 64; h++) tma_load_2d(sB + h * 8192, g.tmB, full, n0 + h * 64, k0);
          }
        }
      }
      if (ok) take_early_ticket(et);     // every copy of the task is on its way: this thread has nothing left to do but the closing barrier
      if (aborted(st)) {       // giving up: wait (bounded) until the copies this task issued into our shared memory have landed
        const uint32_t issued = sc - gp.stage_count[W];
        for (uint32_t i = 0; i < issued && i < (uint32_t)STAGES; i++) {
          const uint32_t c = sc - 1 - i; const int s = c % STAGES; const uint32_t use = c / STAGES;
          for (int spin = 0; spin < 100000; spin++) if (mbar_try(bar_full<BN>(base, s), use & 1)) break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {                                                           // ---- MMA issuer
      uint32_t sc = gp.stage_count[W], tc = gp.tile_count[W];
      bool ok = true;
      for (int t = 0; t < nt && ok; t++, tc++) {
        const int b = tc % CF::NBUF; const uint32_t use = tc / CF::NBUF;
        if (!mbar_wait(bar_acce<BN>(base, b), (use & 1) ^ 1, st)) { if (!aborted(st)) raise_abort(st, ST_MBAR_ACC_TIMEOUT, phase_id, task, 100 + t); ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = gp.tmem_base + (uint32_t)(b * BN);
        for (int kt = 0; kt < KT; kt++, sc++) {
          const int s = sc % STAGES; const uint32_t suse = sc / STAGES;
          if (!mbar_wait(bar_full<BN>(base, s), suse & 1, st)) { if (!aborted(st)) raise_abort(st, ST_MBAR_FULL_TIMEOUT, phase_id, task, kt); ok = false; break; }
          tc_fence_after();
          const uint32_t sA = base + s * CF::STAGE_BYTES, sB = sA + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; kk++) {
            const u64 da = A_MN ? umma_smem_desc(sA + kk * 2048, 8192, 1024) : umma_smem_desc(sA + kk * 32, 16, 1024);
            const u64 db = B_MN ? umma_smem_desc(sB + kk * 2048, 8192, 1024) : umma_smem_desc(sB + kk * 32, 16, 1024);
            umma_bf16(d_tmem, da, db, IDESC, (kt > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(bar_empty<BN>(base, s));       // stage s reusable once these MMAs retire
        }
        if (ok) umma_commit(bar_accf<BN>(base, b));  // accumulator b complete
      }
    }
  } else if (warp >= 4) {                                                      // ---- epilogue warps
    const int e = warp - 4;                      // TMEM lane quadrant == warp % 4
    float* stg = reinterpret_cast<float*>(smem + PIPE_BYTES + e * 4096);
    uint32_t tc = gp.tile_count[W];
    bool ok = true;
    const int cg = lane & 3;
    for (int t = 0; t < nt && ok; t++, tc++) {
      const int b = tc % CF::NBUF; const uint32_t use = tc / CF::NBUF;
      const int n0 = (tn0 + t) * BN;
#pragma unroll
      for (int half = 0; half < BN / 128; half++) {          // 128 columns at a time
        // Epilogues that read `aux` (residual, pre-activation) fetch this thread's 16 row segments of the 128 columns BEFORE
        // waiting for the accumulator, so the loads travel while the MMAs run instead of being 16 dependent round trips.
        uint4 auxr[HAS_AUX_IN ? 16 : 1];
        if constexpr (EPI == GE_DR) {                    // layout of the bf16-staged pass below: row = it*4 + lane/8, 8 columns at (lane%8)*8
          const bf16* aux = reinterpret_cast<const bf16*>(g.aux);
#pragma unroll
          for (int cp = 0; cp < 2; cp++)
#pragma unroll
            for (int it = 0; it < 8; it++)
              auxr[cp * 8 + it] = *reinterpret_cast<const uint4*>(aux + (size_t)(m0 + e * 32 + it * 4 + (lane >> 3)) * g.ldaux + n0 + half * 128 + cp * 64 + (lane & 7) * 8);
        } else if constexpr (HAS_AUX_IN) {
          const bf16* aux = reinterpret_cast<const bf16*>(g.aux);
#pragma unroll
          for (int c = 0; c < 4; c++)
#pragma unroll
            for (int it = 0; it < 4; it++)
              auxr[c * 4 + it] = *reinterpret_cast<const uint4*>(aux + (size_t)(m0 + e * 32 + it * 8 + (lane >> 2)) * g.ldaux + n0 + half * 128 + c * 32 + cg * 8);
        }
        if (half == 0) {
          if (!mbar_wait(bar_accf<BN>(base, b), use & 1, st)) { if (lane == 0 && !aborted(st)) raise_abort(st, ST_MBAR_ACC_TIMEOUT, phase_id, task, t); ok = false; }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after();
        }
        if constexpr (BF16_STAGED) {
          // The stored value is the bf16 rounding of the accumulator itself, so the accumulator is rounded BEFORE the transpose:
          // the thread that owns row `lane` packs 64 columns into eight 16-byte chunks of a 32 x 128 B tile (chunk j at
          // position j ^ (lane & 7)), and the warp reads it back as 4 rows x 128 B per instruction - whole lines for the
          // stores, half the shared-memory traffic of an fp32 transpose (the pipeline's own traffic nearly saturates it).
          unsigned char* sb = reinterpret_cast<unsigned char*>(stg);
          const int sub = lane >> 3, ch = lane & 7;
          float lm[EPI == GE_LSE ? 8 : 1], ls[EPI == GE_LSE ? 8 : 1];   // GE_LSE: running maximum (log2 domain) and sum of 2^(x - max) per row slot
#pragma unroll
          for (int i = 0; i < (EPI == GE_LSE ? 8 : 1); i++) { lm[i] = -INFINITY; ls[i] = 0.f; }
#pragma unroll
          for (int cp = 0; cp < 2; cp++) {                 // 64 columns at a time
#pragma unroll
            for (int hc = 0; hc < 2; hc++) {
              uint32_t r[32];
              tmem_ld32(gp.tmem_base + ((uint32_t)(e * 32) << 16) + (uint32_t)(b * BN + half * 128 + cp * 64 + hc * 32), r);
              if (half == BN / 128 - 1 && cp == 1 && hc == 1) {    // all TMEM reads of this accumulator are done: hand it back early
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acce<BN>(base, b));
              }
#pragma unroll
              for (int q = 0; q < 4; q++) {
                uint4 v;
                v.x = pack2f(__uint_as_float(r[8 * q]), __uint_as_float(r[8 * q + 1])); v.y = pack2f(__uint_as_float(r[8 * q + 2]), __uint_as_float(r[8 * q + 3]));
                v.z = pack2f(__uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5])); v.w = pack2f(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7]));
                *reinterpret_cast<uint4*>(sb + lane * 128 + (((hc * 4 + q) ^ (lane & 7)) << 4)) = v;
              }
            }
            __syncwarp();
            float drs[EPI == GE_DR ? 8 : 1];
            // all eight reads first: a global store between two shared-memory reads keeps the compiler from moving the second
            // read up (it cannot rule out aliasing), and the pass would pay eight shared-memory latencies in a row
            uint4 ov[8];
#pragma unroll
            for (int it = 0; it < 8; it++) { const int rr = it * 4 + sub; ov[it] = *reinterpret_cast<const uint4*>(sb + rr * 128 + ((ch ^ (rr & 7)) << 4)); }
#pragma unroll
            for (int it = 0; it < 8; it++) {
              const int rr = it * 4 + sub;
              const uint4 out = ov[it];
              const size_t row = (size_t)(m0 + e * 32 + rr);
              const int col = n0 + half * 128 + cp * 64 + ch * 8;
              if constexpr (EPI == GE_GELU) {
                *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(g.aux) + row * g.ldaux + col) = out;   // bf16-rounded pre-activation is what backward sees
                float pv[8]; unpack8(out, pv);
#pragma unroll
                for (int i = 0; i < 8; i++) pv[i] = gelu_fwd<true>(pv[i]);
                *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(g.C) + row * g.ldc + col) = pack8(pv);
              } else {
                *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(g.C) + row * g.ldc + col) = out;
              }
              if constexpr (EPI == GE_LSE) {
                float y[8]; unpack8(out, y);               // the STORED values: the partials describe exactly what cross-entropy will read
                float gm = y[0];
#pragma unroll
                for (int i = 1; i < 8; i++) gm = fmaxf(gm, y[i]);
                gm *= 1.4426950408889634f;
                if (gm > lm[it]) { ls[it] *= ex2_approx(lm[it] - gm); lm[it] = gm; }
                float s2 = 0.f;
#pragma unroll
                for (int i = 0; i < 8; i += 2) { ls[it] += ex2_approx(fmaf(y[i], 1.4426950408889634f, -lm[it])); s2 += ex2_approx(fmaf(y[i + 1], 1.4426950408889634f, -lm[it])); }
                ls[it] += s2;
              }
              if constexpr (EPI == GE_DR) {
                float c8[8], o8[8]; unpack8(out, c8); unpack8(auxr[cp * 8 + it], o8);
                float sdot = 0.f;
#pragma unroll
                for (int i = 0; i < 8; i++) sdot = fmaf(c8[i], o8[i], sdot);
                drs[it] = sdot;
              }
            }
            if constexpr (EPI == GE_DR) {                  // one pass = the 64 columns of one head; a row's share sits in 8 lanes
              // the 128 rows of a tile belong to one sequence (the context length is a multiple of 128): one division per tile
              const int bseq = m0 / g.dr_T, t0 = m0 - bseq * g.dr_T + e * 32 + sub;
              float* drow = g.dr + ((size_t)bseq * g.dr_H + (n0 + half * 128) / 64 + cp) * g.dr_T + t0;
#pragma unroll
              for (int it = 0; it < 8; it++) {
                float v = drs[it];
                v += __shfl_xor_sync(0xffffffffu, v, 1); v += __shfl_xor_sync(0xffffffffu, v, 2); v += __shfl_xor_sync(0xffffffffu, v, 4);
                if (ch == 0) drow[it * 4] = v;
              }
            }
            __syncwarp();
          }
          if constexpr (EPI == GE_LSE) {                   // a row's 128 columns sit in 8 lanes: merge their (max, sum) pairs, same result in all eight
            float2* part = reinterpret_cast<float2*>(g.dr) + (size_t)(m0 + e * 32 + sub) * (g.N / 128) + (n0 + half * 128) / 128;
#pragma unroll
            for (int it = 0; it < 8; it++) {
              float m_ = lm[it], s_ = ls[it];
#pragma unroll
              for (int o = 1; o <= 4; o <<= 1) {
                const float mo = __shfl_xor_sync(0xffffffffu, m_, o), so = __shfl_xor_sync(0xffffffffu, s_, o);
                const float mn = fmaxf(m_, mo);
                s_ = s_ * ex2_approx(m_ - mn) + so * ex2_approx(mo - mn);
                m_ = mn;
              }
              if (ch == 0) part[(size_t)it * 4 * (g.N / 128)] = make_float2(m_, s_);
            }
          }
        } else {
#pragma unroll
        for (int c = 0; c < 4; c++) {
          uint32_t r[32];
          tmem_ld32(gp.tmem_base + ((uint32_t)(e * 32) << 16) + (uint32_t)(b * BN + half * 128 + c * 32), r);
          if (half == BN / 128 - 1 && c == 3) {    // all TMEM reads of this accumulator are done: hand it back early
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acce<BN>(base, b));
          }
          // thread = row `lane` of the 32x32 block; 16-byte chunk j goes to position j ^ (lane & 7)
#pragma unroll
          for (int j = 0; j < 8; j++)
            *reinterpret_cast<float4*>(stg + lane * 32 + ((j ^ (lane & 7)) << 2)) =
                make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
          __syncwarp();
          // 8 rows per instruction: lane -> (row = it*8 + lane/4, 8 consecutive columns (lane%4)*8..)
          float4 av[8];                            // all reads before the first global store (see the bf16-staged pass)
#pragma unroll
          for (int it = 0; it < 4; it++) {
            const int rr = it * 8 + (lane >> 2);
            av[2 * it] = *reinterpret_cast<const float4*>(stg + rr * 32 + (((2 * cg) ^ (rr & 7)) << 2));
            av[2 * it + 1] = *reinterpret_cast<const float4*>(stg + rr * 32 + (((2 * cg + 1) ^ (rr & 7)) << 2));
          }
#pragma unroll
          for (int it = 0; it < 4; it++) {
            const int rr = it * 8 + (lane >> 2);
            const float4 a0 = av[2 * it], a1 = av[2 * it + 1];
            const float acc[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            epi_store8<EPI>(g, (size_t)(m0 + e * 32 + rr), n0 + half * 128 + c * 32 + cg * 8, acc, auxr[HAS_AUX_IN ? c * 4 + it : 0]);
          }
          __syncwarp();
        }
        }
      }
    }
  }
  gp.stage_count[W] += (uint32_t)(nt * KT);
  gp.tile_count[W] += (uint32_t)nt;
  __syncthreads();
}

template <int LAYOUT, int EPI>
__device__ __forceinline__ void dispatch_bn(const PhaseDesc& d, int task, unsigned char* smem, GemmPipe& gp, DevStatus* st, int phase_id, const EarlyTicket& et) {
  if (d.g.bn == 256) gemm_tc_task<LAYOUT, EPI, 256>(d.g, d.tiles_m, task, smem, gp, st, phase_id, et, d.i0);
  else gemm_tc_task<LAYOUT, EPI, 128>(d.g, d.tiles_m, task, smem, gp, st, phase_id, et, d.i0);
}
// run-time dispatch over the (layout, epilogue) pairs the training graph uses
__device__ __noinline__ void run(const PhaseDesc& d, int task, unsigned char* smem, GemmPipe& gp, DevStatus* st, int phase_id, const EarlyTicket& et) {
  switch (d.layout * 8 + d.epi) {
    case GL_NN * 8 + GE_STORE: dispatch_bn<GL_NN, GE_STORE>(d, task, smem, gp, st, phase_id, et); break;
    case GL_NN * 8 + GE_RES:   dispatch_bn<GL_NN, GE_RES>(d, task, smem, gp, st, phase_id, et); break;
    case GL_NN * 8 + GE_GELU:  dispatch_bn<GL_NN, GE_GELU>(d, task, smem, gp, st, phase_id, et); break;
    case GL_NN * 8 + GE_F32:   dispatch_bn<GL_NN, GE_F32>(d, task, smem, gp, st, phase_id, et); break;      // split-K partial products
    case GL_NT * 8 + GE_STORE: dispatch_bn<GL_NT, GE_STORE>(d, task, smem, gp, st, phase_id, et); break;
    case GL_NT * 8 + GE_DGELU: dispatch_bn<GL_NT, GE_DGELU>(d, task, smem, gp, st, phase_id, et); break;
    case GL_NT * 8 + GE_DR:    gemm_tc_task<GL_NT, GE_DR, 128>(d.g, d.tiles_m, task, smem, gp, st, phase_id, et, d.i0); break;
    case GL_NT * 8 + GE_LSE:   gemm_tc_task<GL_NT, GE_LSE, 128>(d.g, d.tiles_m, task, smem, gp, st, phase_id, et, d.i0); break;
    case GL_TN * 8 + GE_F32:   dispatch_bn<GL_TN, GE_F32>(d, task, smem, gp, st, phase_id, et); break;
    case GL_TN * 8 + GE_STORE: dispatch_bn<GL_TN, GE_STORE>(d, task, smem, gp, st, phase_id, et); break;
    default: if (threadIdx.x == 0) raise_abort(st, ST_BAD_DESC, phase_id, task, d.layout * 8 + d.epi); __syncthreads(); break;
  }
}

}  // namespace gemm_tc
}  // namespace ofa
