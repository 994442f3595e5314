// bf16 tensor-core GEMM task for sm_100a: TMA -> swizzled shared memory -> tcgen05.mma -> TMEM -> epilogue.
//
// Task contract (replaces the reference's `tg::tile<LAYOUT,EPI>` = gemm::sm100::tile_tc,
// llm/b200/gemm_tcgen05/gemm_sm100.cuh:174-289, with the layouts/epilogues of llm/gemm/gemm.cuh:18-50):
//   one task = a STRIP of `nsub` consecutive 128x128 tiles of C that share their 128 rows; all 256 threads call
//   gemm_tc_task() together. Differences in design from the reference tile:
//     * the mbarriers and the 256 TMEM columns of a block live for the whole kernel; phase parities are derived from
//       running counters kept in `GemmPipe`, so nothing is re-initialised or invalidated between tiles or tasks;
//     * inside a strip the TMA producer (warp 0) and the MMA issuer (warp 1) run ahead of the epilogue: the
//       accumulator is double-buffered in TMEM (2 x 128 columns) and drained by warps 4..7 while the next tile's MMAs
//       are in flight, so only the first fill and the last drain of a strip are exposed;
//     * the epilogue never touches the pipeline buffers: each epilogue warp transposes 32x32 fp32 blocks through its own
//       4 KB staging area (XOR-swizzled, conflict-free) and then moves whole 64/128-byte row segments to global memory;
//     * every wait is bounded and aborts the grid cleanly on expiry.
//   K order is fixed (k ascending, one accumulator) => results are deterministic and independent of the schedule.
//
// Operand staging (SWIZZLE_128B everywhere, one pipeline stage = 64 values of K for a 128x128 tile = 32 KB):
//   K-major operand  X[rows][K]  (A of NN/NT, B of NT): one TMA box {64 k, 128 rows} -> 128 rows x 128 B; UMMA descriptor
//     SBO = 1024 B (8 rows), a step of 16 in K advances the start address by 32 B.
//   MN-major operand X[K][cols]  (B of NN/TN, A of TN): two TMA boxes {64 cols, 64 k}, 8 KB apart -> per box 64 k-rows x
//     128 B; UMMA descriptor LBO = 8192 B (between the two 64-wide halves), SBO = 1024 B (8 k-rows), a step of 16 in K
//     advances the start address by 2048 B.
#pragma once
#include "common.cuh"
#include "task_api.h"

namespace ofa {
namespace gemm_tc {

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int STAGES = 3;
constexpr int OPERAND_BYTES = 128 * BK * 2;          // 16 KB
constexpr int STAGE_BYTES = 2 * OPERAND_BYTES;       // 32 KB
constexpr int PIPE_BYTES = STAGES * STAGE_BYTES;     // 96 KB
constexpr int EPI_WARPS = 4;                         // warps 4..7
constexpr int STAGING_BYTES = EPI_WARPS * 32 * 32 * 4;   // 16 KB
constexpr int BAR_OFFSET = PIPE_BYTES + STAGING_BYTES;   // barriers + TMEM slot live behind everything else
constexpr int BAR_BYTES = 256;
constexpr int SMEM_BYTES = BAR_OFFSET + BAR_BYTES;   // 114,944 B: two blocks per SM
constexpr int TMEM_COLS = 256;                       // two 128-column fp32 accumulators

// barrier slots (8 bytes each) at smem + BAR_OFFSET
//   full[s]  : TMA bytes of stage s landed            (count 1 + tx)
//   empty[s] : the MMAs reading stage s completed      (count 1, tcgen05.commit)
//   accf[b]  : accumulator b complete                  (count 1, tcgen05.commit)
//   acce[b]  : accumulator b drained by the epilogue   (count EPI_WARPS)
__device__ __forceinline__ uint32_t bar_full(uint32_t base, int s) { return base + BAR_OFFSET + 8u * s; }
__device__ __forceinline__ uint32_t bar_empty(uint32_t base, int s) { return base + BAR_OFFSET + 8u * (STAGES + s); }
__device__ __forceinline__ uint32_t bar_accf(uint32_t base, int b) { return base + BAR_OFFSET + 8u * (2 * STAGES + b); }
__device__ __forceinline__ uint32_t bar_acce(uint32_t base, int b) { return base + BAR_OFFSET + 8u * (2 * STAGES + 2 + b); }
constexpr int TMEM_SLOT_OFFSET = BAR_OFFSET + 8 * (2 * STAGES + 4);

// Per-thread running counters; every thread advances all of them identically at the end of a task.
struct GemmPipe {
  uint32_t stage_count;   // pipeline stages produced/consumed since block start
  uint32_t tile_count;    // accumulator tiles since block start
  uint32_t tmem_base;
};

// Once per block, before its first GEMM task. All 256 threads. Returns false (and aborts) if shared memory is misaligned.
__device__ __forceinline__ bool block_init(GemmPipe& gp, unsigned char* smem, DevStatus* st) {
  const uint32_t base = smem_u32(smem);
  gp.stage_count = 0; gp.tile_count = 0; gp.tmem_base = 0;
  const bool ok = (base & 1023u) == 0;
  if (!ok) { if (threadIdx.x == 0) raise_abort(st, ST_SMEM_MISALIGNED, -1, -1, (int)base); }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(bar_full(base, s), 1); mbar_init(bar_empty(base, s), 1); }
    for (int b = 0; b < 2; b++) { mbar_init(bar_accf(base, b), 1); mbar_init(bar_acce(base, b), EPI_WARPS); }
    mbar_fence_init();
  }
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
  const uint32_t base = smem_u32(smem);
  (void)base;
  if (aborted(st)) __nanosleep(20000);   // copies issued by a task that bailed out were already drained there; this covers the rest
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x < 32) tmem_dealloc(gp.tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------- epilogue math
template <int EPI>
__device__ __forceinline__ void epi_store8(const GemmArgs& g, size_t row, int col, const float* acc) {
  if constexpr (EPI == GE_F32) {
    float* dst = reinterpret_cast<float*>(g.C) + row * g.ldc + col;
    float4 v0 = make_float4(acc[0], acc[1], acc[2], acc[3]), v1 = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if (g.accumulate) {
      const float4 o0 = *reinterpret_cast<const float4*>(dst), o1 = *reinterpret_cast<const float4*>(dst + 4);
      v0.x += o0.x; v0.y += o0.y; v0.z += o0.z; v0.w += o0.w; v1.x += o1.x; v1.y += o1.y; v1.z += o1.z; v1.w += o1.w;
    }
    *reinterpret_cast<float4*>(dst) = v0; *reinterpret_cast<float4*>(dst + 4) = v1;
  } else {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = acc[i];
    bf16* C = reinterpret_cast<bf16*>(g.C);
    bf16* aux = reinterpret_cast<bf16*>(g.aux);
    if constexpr (EPI == GE_RES) {
      float r[8]; ldv(aux + row * g.ldaux + col, r);
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] += r[i];
    } else if constexpr (EPI == GE_GELU) {
      const uint4 pre = pack8(v);                                   // bf16-rounded pre-activation is what backward sees
      *reinterpret_cast<uint4*>(aux + row * g.ldaux + col) = pre;
      float p[8]; unpack8(pre, p);
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] = gelu_fwd<true>(p[i]);
    } else if constexpr (EPI == GE_DGELU) {
      float p[8]; ldv(aux + row * g.ldaux + col, p);
#pragma unroll
      for (int i = 0; i < 8; i++) v[i] *= gelu_bwd<true>(p[i]);
    }
    *reinterpret_cast<uint4*>(C + row * g.ldc + col) = pack8(v);
  }
}

// ---------------------------------------------------------------------------------------------- the task
// task index -> (tile_m, first tile_n): consecutive tasks walk down M first so that neighbouring blocks share the B strip.
template <int LAYOUT, int EPI>
__device__ __forceinline__ void gemm_tc_task(const GemmArgs& g, int tiles_m, int task, unsigned char* smem, GemmPipe& gp,
                                             DevStatus* st, int phase_id) {
  constexpr bool A_MN = (LAYOUT == GL_TN), B_MN = (LAYOUT != GL_NT);
  constexpr uint32_t IDESC = umma_idesc(A_MN, B_MN, BM, BN);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t base = smem_u32(smem);
  const int KT = g.K / BK;
  const int tiles_n = g.N / BN;
  const int tm = task % tiles_m, strip = task / tiles_m;
  const int tn0 = strip * g.nsub;
  const int nt = min(g.nsub, tiles_n - tn0);
  const int m0 = tm * BM;

  if (warp == 0) {
    if (lane == 0) {                                                           // ---- TMA producer
      fence_proxy_async();     // operands were written with ordinary stores by earlier phases (possibly other SMs)
      uint32_t sc = gp.stage_count;
      bool ok = true;
      for (int t = 0; t < nt && ok; t++) {
        const int n0 = (tn0 + t) * BN;
        for (int kt = 0; kt < KT; kt++, sc++) {
          const int s = sc % STAGES; const uint32_t use = sc / STAGES;
          if (!mbar_wait(bar_empty(base, s), (use & 1) ^ 1, st)) { if (!aborted(st)) raise_abort(st, ST_MBAR_EMPTY_TIMEOUT, phase_id, task, kt); ok = false; break; }
          mbar_expect_tx(bar_full(base, s), STAGE_BYTES);
          const uint32_t sA = base + s * STAGE_BYTES, sB = sA + OPERAND_BYTES;
          const int k0 = kt * BK;
          if (!A_MN) tma_load_2d(sA, g.tmA, bar_full(base, s), k0, m0);
          else { tma_load_2d(sA, g.tmA, bar_full(base, s), m0, k0); tma_load_2d(sA + 8192, g.tmA, bar_full(base, s), m0 + 64, k0); }
          if (!B_MN) tma_load_2d(sB, g.tmB, bar_full(base, s), k0, n0);
          else { tma_load_2d(sB, g.tmB, bar_full(base, s), n0, k0); tma_load_2d(sB + 8192, g.tmB, bar_full(base, s), n0 + 64, k0); }
        }
      }
      if (aborted(st)) {       // giving up: wait (bounded) until the copies this task issued into our shared memory have landed
        const uint32_t issued = sc - gp.stage_count;
        for (uint32_t i = 0; i < issued && i < (uint32_t)STAGES; i++) {
          const uint32_t c = sc - 1 - i; const int s = c % STAGES; const uint32_t use = c / STAGES;
          for (int spin = 0; spin < 100000; spin++) if (mbar_try(bar_full(base, s), use & 1)) break;
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {                                                           // ---- MMA issuer
      uint32_t sc = gp.stage_count, tc = gp.tile_count;
      bool ok = true;
      for (int t = 0; t < nt && ok; t++, tc++) {
        const int b = tc & 1; const uint32_t use = tc >> 1;
        if (!mbar_wait(bar_acce(base, b), (use & 1) ^ 1, st)) { if (!aborted(st)) raise_abort(st, ST_MBAR_ACC_TIMEOUT, phase_id, task, 100 + t); ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = gp.tmem_base + (uint32_t)(b * BN);
        for (int kt = 0; kt < KT; kt++, sc++) {
          const int s = sc % STAGES; const uint32_t suse = sc / STAGES;
          if (!mbar_wait(bar_full(base, s), suse & 1, st)) { if (!aborted(st)) raise_abort(st, ST_MBAR_FULL_TIMEOUT, phase_id, task, kt); ok = false; break; }
          tc_fence_after();
          const uint32_t sA = base + s * STAGE_BYTES, sB = sA + OPERAND_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / 16; kk++) {
            const u64 da = A_MN ? umma_smem_desc(sA + kk * 2048, 8192, 1024) : umma_smem_desc(sA + kk * 32, 16, 1024);
            const u64 db = B_MN ? umma_smem_desc(sB + kk * 2048, 8192, 1024) : umma_smem_desc(sB + kk * 32, 16, 1024);
            umma_bf16(d_tmem, da, db, IDESC, (kt > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(bar_empty(base, s));       // stage s reusable once these MMAs retire
        }
        if (ok) umma_commit(bar_accf(base, b));  // accumulator b complete
      }
    }
  } else if (warp >= 4) {                                                      // ---- epilogue warps
    const int e = warp - 4;                      // TMEM lane quadrant == warp % 4
    float* stg = reinterpret_cast<float*>(smem + PIPE_BYTES + e * 4096);
    uint32_t tc = gp.tile_count;
    bool ok = true;
    for (int t = 0; t < nt && ok; t++, tc++) {
      const int b = tc & 1; const uint32_t use = tc >> 1;
      if (!mbar_wait(bar_accf(base, b), use & 1, st)) { if (lane == 0 && !aborted(st)) raise_abort(st, ST_MBAR_ACC_TIMEOUT, phase_id, task, t); ok = false; }
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int n0 = (tn0 + t) * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; c++) {
        uint32_t r[32];
        tmem_ld32(gp.tmem_base + ((uint32_t)(e * 32) << 16) + (uint32_t)(b * BN + c * 32), r);
        if (c == BN / 32 - 1) {                  // all TMEM reads of this accumulator are done: hand it back early
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_acce(base, b));
        }
        // thread = row `lane` of the 32x32 block; 16-byte chunk j goes to position j ^ (lane & 7)
#pragma unroll
        for (int j = 0; j < 8; j++)
          *reinterpret_cast<float4*>(stg + lane * 32 + ((j ^ (lane & 7)) << 2)) =
              make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        __syncwarp();
        // 8 rows per instruction: lane -> (row = it*8 + lane/4, 8 consecutive columns (lane%4)*8..)
        const int cg = lane & 3;
#pragma unroll
        for (int it = 0; it < 4; it++) {
          const int rr = it * 8 + (lane >> 2);
          const float4 a0 = *reinterpret_cast<const float4*>(stg + rr * 32 + (((2 * cg) ^ (rr & 7)) << 2));
          const float4 a1 = *reinterpret_cast<const float4*>(stg + rr * 32 + (((2 * cg + 1) ^ (rr & 7)) << 2));
          const float acc[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
          epi_store8<EPI>(g, (size_t)(m0 + e * 32 + rr), n0 + c * 32 + cg * 8, acc);
        }
        __syncwarp();
      }
    }
  }
  gp.stage_count += (uint32_t)(nt * KT);
  gp.tile_count += (uint32_t)nt;
  __syncthreads();
}

// run-time dispatch over the (layout, epilogue) pairs the training graph uses
__device__ __noinline__ void run(const PhaseDesc& d, int task, unsigned char* smem, GemmPipe& gp, DevStatus* st, int phase_id) {
  switch (d.layout * 8 + d.epi) {
    case GL_NN * 8 + GE_STORE: gemm_tc_task<GL_NN, GE_STORE>(d.g, d.tiles_m, task, smem, gp, st, phase_id); break;
    case GL_NN * 8 + GE_RES:   gemm_tc_task<GL_NN, GE_RES>(d.g, d.tiles_m, task, smem, gp, st, phase_id); break;
    case GL_NN * 8 + GE_GELU:  gemm_tc_task<GL_NN, GE_GELU>(d.g, d.tiles_m, task, smem, gp, st, phase_id); break;
    case GL_NT * 8 + GE_STORE: gemm_tc_task<GL_NT, GE_STORE>(d.g, d.tiles_m, task, smem, gp, st, phase_id); break;
    case GL_NT * 8 + GE_DGELU: gemm_tc_task<GL_NT, GE_DGELU>(d.g, d.tiles_m, task, smem, gp, st, phase_id); break;
    case GL_TN * 8 + GE_F32:   gemm_tc_task<GL_TN, GE_F32>(d.g, d.tiles_m, task, smem, gp, st, phase_id); break;
    case GL_TN * 8 + GE_STORE: gemm_tc_task<GL_TN, GE_STORE>(d.g, d.tiles_m, task, smem, gp, st, phase_id); break;
    default: if (threadIdx.x == 0) raise_abort(st, ST_BAD_DESC, phase_id, task, d.layout * 8 + d.epi); __syncthreads(); break;
  }
}

}  // namespace gemm_tc
}  // namespace ofa
