// The persistent kernel: one launch, blocks that never exit until their job is finished, on-GPU ticket queues with
// dependency counters, and a static split of the SMs between the training job, the serving (decode) job and a reserved
// idle partition.
//
// Scheduling model (same contract as the reference's job_loop / ofa_kernel, llm/b200/megakernel/ofa.cu:220-326):
//   thread 0 of a block takes the next ticket g of its job with one fetch-add; g -> (step, phase, task) through the prefix
//   table; it then waits until every dependency (phase p, step delta d) satisfies done[p] >= ntasks[p]*(step+1+d); the
//   whole block runs the task; after a device-scope fence thread 0 bumps done[phase]. Phases are topologically ordered and
//   cross-step dependencies point backwards, so every dependency is a lower ticket and the lowest unfinished ticket is
//   always runnable: no deadlock as long as every claimed ticket is eventually run, which holds because a block holds at
//   most one ticket.
// What differs from the reference: the phase lookup is a binary search; every wait is bounded (%globaltimer deadline and a
// grid-wide abort word) so that a wedged task makes the kernel RETURN with a status instead of hanging the GPU; the
// per-block tensor-core state (mbarriers, TMEM) is created once per block, not per task; external (host / other-rank)
// events enter the graph as ordinary 1-task phases (TK_EXT_WAIT / TK_EXT_SIGNAL).
#pragma once
#include "common.cuh"
#include "task_api.h"
#include "elementwise.cuh"
#include "gemm_tc.cuh"
#include "attn_common.cuh"
#include "attn_tc.cuh"
#include "simt_f32.cuh"
#include "decode.cuh"
#include <type_traits>

namespace ofa {

template <class T> struct IsBf16 { static constexpr bool value = std::is_same<T, bf16>::value; };

// ---------------------------------------------------------------------------------------------- one training task
template <class T, int D, int DH>
__device__ __forceinline__ void run_train_task(const Ctx& C, const PhaseDesc& d, int ph, int local, int step, unsigned char* smem,
                                               gemm_tc::GemmPipe& gp, attn_tc::AttnPipe& ap, uint32_t& bulk_uses, uint32_t& adam_tiles, uint32_t& ce_chunks,
                                               const EarlyTicket& et) {
  const ModelDims& md = C.md;
  switch (d.kind) {
    case TK_DATA:
      ew::data_task(local, step + C.step_base, C.data, C.ntok, C.starts, C.nstarts, C.seed, C.tok_in, C.tok_tgt, md.T, md.B);
      break;
    case TK_EMBED:
      ew::embed_fwd_task<T, D>(local, (T*)d.p[0], (const T*)d.p[1], (const T*)d.p[2], (const int*)d.p[3], md.N, md.T);
      break;
    case TK_LN_FWD:
      ew::ln_fwd_task<T, D>(local, (T*)d.p[0], (float*)d.p[1], (float*)d.p[2], (const T*)d.p[3], (const T*)d.p[4], md.N);
      break;
    case TK_GEMM:
      if constexpr (IsBf16<T>::value) gemm_tc::run(d, local, smem, gp, C.status, ph, et);
      else f32::gemm_run(d, local, smem);
      break;
    case TK_ATT_FWD: {
      if constexpr (IsBf16<T>::value) {
        const int BH = md.B * md.H, QT = md.T / attn::QTILE;
        const int qt = QT - 1 - local / BH, bh = local % BH;      // heavy (late) query tiles first
        attn_tc::fwd_task((const attn_tc::Maps*)d.p[6], (bf16*)d.p[1], (float*)d.p[2], bh / md.H, bh % md.H, qt, md.T, md.H, smem, ap, gp.tmem_base, C.status, ph, local, et);
      } else {
        f32::attn_fwd_task<DH>((const float*)d.p[0], (float*)d.p[1], (float*)d.p[2], local / md.H, local % md.H, md.T, md.H, smem);
      }
      break;
    }
    case TK_ATT_PREP: {
      if constexpr (IsBf16<T>::value) {
        const int BH = md.B * md.H;
        const int rt = local / BH, bh = local % BH;
        attn::bwd_prep_task((const bf16*)d.p[0], (const bf16*)d.p[1], (float*)d.p[2], bh / md.H, bh % md.H, rt, md.T, md.H);
      }
      break;
    }
    case TK_ATT_BWD: {
      if constexpr (IsBf16<T>::value) {
        const int BH = md.B * md.H, QT = md.T / attn::QTILE;
        if (local < BH * QT) {                                     // dK/dV: early key tiles see the most queries -> first
          const int kt = local / BH, bh = local % BH;
          attn_tc::bwd_dkdv_task((const attn_tc::Maps*)d.p[6], (const float*)d.p[2], (const float*)d.p[3], (bf16*)d.p[4], bh / md.H, bh % md.H, kt, md.T, md.H, smem, ap, gp.tmem_base, C.status, ph, local, et);
        } else {                                                   // dQ: late query tiles see the most keys -> first
          const int l2 = local - BH * QT, qt = QT - 1 - l2 / BH, bh = l2 % BH;
          attn_tc::bwd_dq_task((const attn_tc::Maps*)d.p[6], (const float*)d.p[2], (const float*)d.p[3], (bf16*)d.p[4], bh / md.H, bh % md.H, qt, md.T, md.H, smem, ap, gp.tmem_base, C.status, ph, local, et);
        }
      } else {
        f32::attn_bwd_task<DH>((const float*)d.p[0], (const float*)d.p[5], (const float*)d.p[1], (const float*)d.p[2], (float*)d.p[4],
                               local / md.H, local % md.H, md.T, md.H, smem);
      }
      break;
    }
    case TK_CE:
      if constexpr (IsBf16<T>::value) {
        if (d.p[3] && md.V % 8 == 0) {                 // the LM-head GEMM left softmax partials: one streamed pass over the logits
          ew::ce_task_stream(local, (bf16*)d.p[0], (const int*)d.p[1], (float*)d.p[2], (const float2*)d.p[3], d.i2, md.N, md.V, 1.0f / (float)md.N, smem,
                             smem_u32(smem + C.smem_bytes - CTRL_BYTES + 112), smem_u32(smem + C.smem_bytes - CTRL_BYTES + 160), ce_chunks, C.status);
          break;
        }
        if ((size_t)md.V * 2 <= (size_t)d.i0 && md.V % 8 == 0) {
          ew::ce_task_bulk(local, (bf16*)d.p[0], (const int*)d.p[1], (float*)d.p[2], md.N, md.V, 1.0f / (float)md.N, smem,
                           smem_u32(smem + C.smem_bytes - CTRL_BYTES + 104), bulk_uses, C.status);
          break;
        }
      }
      ew::ce_task<T>(local, (T*)d.p[0], (const int*)d.p[1], (float*)d.p[2], md.N, md.V, 1.0f / (float)md.N, smem, d.i0);
      break;
    case TK_CE_MEAN: {
      const float lv = ew::ce_mean_task((float*)d.p[0], (const float*)d.p[1], md.N, smem);
      if (threadIdx.x == 0) { C.loss_hist[step] = lv; if (C.live) C.live->loss = lv; }
      break;
    }
    case TK_LN_BWD:
      ew::ln_bwd_task<T, D>(local, (T*)d.p[0], (float*)d.p[1], (const T*)d.p[2], (const T*)d.p[3], (const float*)d.p[4],
                            (const float*)d.p[5], (const T*)d.p[6], (const T*)d.p[7], md.N, smem);
      break;
    case TK_LN_DG:
      if (d.i1) ew::ln_dgamma_reduce_task<bf16>(local, (bf16*)d.p[0], (const float*)d.p[1], (md.N + ew::ROWS_PER_TASK - 1) / ew::ROWS_PER_TASK, D, d.i0);
      else ew::ln_dgamma_reduce_task<float>(local, (float*)d.p[0], (const float*)d.p[1], (md.N + ew::ROWS_PER_TASK - 1) / ew::ROWS_PER_TASK, D, d.i0);
      break;
    case TK_EMB_WTE:
      if (d.i1) ew::embed_bwd_wte_task<T, D, bf16>(local, (bf16*)d.p[0], (const T*)d.p[1], (const int*)d.p[2], md.N, md.V, d.i0, smem);
      else ew::embed_bwd_wte_task<T, D, float>(local, (float*)d.p[0], (const T*)d.p[1], (const int*)d.p[2], md.N, md.V, d.i0, smem);
      break;
    case TK_EMB_WPE:
      if (d.i1) ew::embed_bwd_wpe_task<T, bf16>(local, (bf16*)d.p[0], (const T*)d.p[1], md.N, md.T, D);
      else ew::embed_bwd_wpe_task<T, float>(local, (float*)d.p[0], (const T*)d.p[1], md.N, md.T, D);
      break;
    case TK_ADAMW: {
      const ew::AdamHP hp = ew::adam_hp(C.hp, step + C.step_base);
      if constexpr (IsBf16<T>::value) {               // inputs staged by the copy engine (the fp32 preset's blocks have no room for the stages)
        const uint32_t bar0 = smem_u32(smem + C.smem_bytes - CTRL_BYTES + 224);
        if (d.i2 == 0) {
          if (d.i1) ew::adamw_task_bulk<T, bf16>(local, (float*)d.p[0], (const bf16*)d.p[1], (float*)d.p[2], (float*)d.p[3], (T*)d.p[4], d.n, hp, (const int2*)d.p[5], d.i0, smem, bar0, adam_tiles, C.status);
          else ew::adamw_task_bulk<T, float>(local, (float*)d.p[0], (const float*)d.p[1], (float*)d.p[2], (float*)d.p[3], (T*)d.p[4], d.n, hp, (const int2*)d.p[5], d.i0, smem, bar0, adam_tiles, C.status);
          break;
        }
      }
      if (d.i1) ew::adamw_task<T, bf16>(local, (float*)d.p[0], (const bf16*)d.p[1], (float*)d.p[2], (float*)d.p[3], (T*)d.p[4], d.n, hp, (const int2*)d.p[5], d.i0);
      else ew::adamw_task<T, float>(local, (float*)d.p[0], (const float*)d.p[1], (float*)d.p[2], (float*)d.p[3], (T*)d.p[4], d.n, hp, (const int2*)d.p[5], d.i0);
      break;
    }
    case TK_SUMCAST:
      ew::sumcast_task<T>(local, (T*)d.p[0], &d.p[1], d.i0, d.n);
      break;
    case TK_EXT_SIGNAL:
      // flag values count steps since the context was created, so a stale value from an earlier launch is always too small
      if (threadIdx.x == 0) { __threadfence_system(); *reinterpret_cast<volatile int*>(d.p[0]) = C.step_base + step + 1; __threadfence_system(); }
      break;
    case TK_EXT_WAIT:
      if (threadIdx.x == 0) {
        const volatile int* flag = reinterpret_cast<const volatile int*>(d.p[0]);
        const u64 t0 = gtimer();
        while (*flag < C.step_base + step + 1) {
          if (aborted(C.status)) break;
          if (gtimer() - t0 > C.dep_timeout_ns) { raise_abort(C.status, ST_EXTERNAL_TIMEOUT, ph, local, step); break; }
          __nanosleep(200);
        }
        __threadfence_system();
      }
      break;
    default: break;   // TK_BARRIER
  }
}

template <class T, int D, int DH>
__device__ __forceinline__ void run_decode_task(const Ctx& C, const PhaseDesc& d, int local, unsigned char* smem, uint32_t bar, uint32_t parity) {
  switch (d.kind) {
    case TK_DEC_QKV: dec::task_qkv<T, D, DH>(C.dp, C.md, d.i0, local, smem, bar, parity, C.status); break;
    case TK_DEC_ATTWO: dec::task_attwo<T, D, DH>(C.dp, C.md, d.i0, local, smem, bar, parity, C.status); break;
    case TK_DEC_UPDN: dec::task_updn<T, D, DH>(C.dp, C.md, d.i0, local, smem, bar, parity, C.status); break;
    case TK_DEC_HEAD: dec::task_head<T, D, DH>(C.dp, C.md, local, smem, bar, parity, C.status); break;
    case TK_DEC_SAMPLE: dec::task_sample<T, D, DH>(C.dp, C.md, C.live, smem); break;
    default: break;
  }
}

// ---------------------------------------------------------------------------------------------- scheduler
// Dependency wait of thread 0 (bounded). Returns 0 when every dependency of (step, ph) is satisfied, -2 when the block must
// leave (job finished elsewhere, abort, or deadline). `R` is the phase's scheduling record (kernel parameter or shared memory).
struct DepSet { int cnt; int ph[4], dl[4], nt[4], gr[4]; int rb_off, rb_map; bool any_rb; };
template <class RecPtr>
__device__ __forceinline__ void load_deps(DepSet& d, RecPtr rec) {      // rec: int-indexable view of a SchedRec
  d.cnt = rec[2]; d.rb_off = rec[4]; d.rb_map = rec[5];
  d.any_rb = false;
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const int w = rec[6 + 2 * k];
    d.ph[k] = w & 0xFFFF; d.dl[k] = (w & DEP_PREV) ? -1 : 0; d.gr[k] = (w & DEP_RB) ? 1 : 0; d.nt[k] = rec[7 + 2 * k];
    d.any_rb = d.any_rb || (k < d.cnt && d.gr[k]);
  }
}
// row block a task writes (prod) and the range of row blocks it reads from its row-block-grain producers [clo, chi]
__device__ __forceinline__ void rb_of_task(int rb_map, const ModelDims& md, int local, int& prod, int& clo, int& chi) {
  const int kind = rb_map & 0xFF, a = rb_map >> 8;
  prod = clo = chi = 0;
  if (kind == RB_MOD) prod = clo = chi = local % a;
  else if (kind == RB_DIV) prod = clo = chi = local / a;
  else if (kind == RB_ATT_FWD) {
    const int BH = md.B * md.H, QT = md.T >> 7;
    const int qt = QT - 1 - local / BH, b = (local % BH) / md.H;
    prod = b * QT + qt; clo = b * QT; chi = prod;
  } else if (kind == RB_ATT_BWD) {
    const int BH = md.B * md.H, QT = md.T >> 7;
    if (local < BH * QT) { const int kt = local / BH, b = (local % BH) / md.H; prod = b * QT + kt; clo = prod; chi = b * QT + QT - 1; }
    else { const int l2 = local - BH * QT, qt = QT - 1 - l2 / BH, b = (l2 % BH) / md.H; prod = clo = chi = b * QT + qt; }
  }
}
__device__ __forceinline__ int wait_deps(const Ctx& C, const Job& J, int job_id, int step, int ph, int local, const DepSet& R, const int* prod_rb_off) {
  const int cnt = R.cnt;
  const u64 t0 = gtimer();
  // a dependency may legitimately sit behind an external wait that is about to give up: its own bound is half as long again, so
  // that the status names the external flag that was never raised and not one of the tasks queued behind it
  const u64 limit = C.dep_timeout_ns + (C.dep_timeout_ns >> 1);
  unsigned spins = 0;
  if (cnt >= 0) {
    // up to four dependencies from the phase's scheduling record: their counters are read with relaxed loads that are all in
    // flight together, and one acquire fence after the last successful check orders the task's reads behind them
    int need[4]; const int* ctr[4]; int span[4];
    int prod = 0, clo = 0, chi = 0;
    if (R.any_rb) rb_of_task(R.rb_map, C.md, local, prod, clo, chi);
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int p = k < cnt ? R.ph[k] : 0, dl = k < cnt ? R.dl[k] : 0, nt = k < cnt ? R.nt[k] : 0;
      const bool g = k < cnt && R.gr[k];
      ctr[k] = g ? J.done_rb + prod_rb_off[k] + clo : J.done + p;
      span[k] = g ? chi - clo + 1 : 1;
      need[k] = k < cnt ? nt * (step + 1 + dl) : 0;
    }
    for (;;) {
      bool ready = true;
#pragma unroll
      for (int k = 0; k < 4; k++) {
        if (need[k] > 0) {
          int v = ld_relaxed(ctr[k]);
          for (int q = 1; q < span[k]; q++) v = min(v, ld_relaxed(ctr[k] + q));
          ready = ready && v >= need[k];
        }
      }
      if (ready) { fence_acquire(); return 0; }
      if (job_id == 1 && C.use_train && ld_relaxed(C.finished)) return -2;
      if ((++spins & 63u) == 0) {
        if (aborted(C.status)) return -2;
        if (gtimer() - t0 > limit) { raise_abort(C.status, ST_DEP_TIMEOUT, ph, local, step); return -2; }
      }
      __nanosleep(job_id == 1 ? 20 : 80);
    }
  }
  const int off = __ldg(J.dep_off + ph), n = __ldg(J.dep_cnt + ph);
  for (;;) {
    bool ready = true;
    for (int k = 0; k < n && ready; k++) {
      const Dep e = J.deps[off + k];
      const int need = __ldg(J.ntasks + e.phase) * (step + 1 + e.delta);
      if (need > 0 && ld_acquire(J.done + e.phase) < need) ready = false;
    }
    if (ready) return 0;
    if (job_id == 1 && C.use_train && ld_relaxed(C.finished)) return -2;
    if ((++spins & 63u) == 0) {
      if (aborted(C.status)) return -2;
      if (gtimer() - t0 > limit) { raise_abort(C.status, ST_DEP_TIMEOUT, ph, local, step); return -2; }
    }
    __nanosleep(job_id == 1 ? 20 : 80);
  }
}

__device__ __forceinline__ void sched_cp16(uint32_t dst, const void* src) { asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void sched_cp_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

template <class T, int D, int DH>
__device__ void job_loop(const Ctx& C, const Job& J, int job_id, unsigned char* smem) {
  unsigned char* ctrl = smem + C.smem_bytes - CTRL_BYTES;   // the last bytes of dynamic shared memory are the block's control area (map in gemm_tc.cuh)
  volatile int* s_sel = reinterpret_cast<volatile int*>(ctrl + 128);
  static_assert(sizeof(PhaseDesc) <= 256 && sizeof(PhaseDesc) % 16 == 0, "descriptor copy does not fit the control area");
  static_assert(sizeof(SchedRec) == 64, "scheduling record is one 64-byte line");
  int slot = 0;                                     // which of the two descriptor slots holds the phase being worked on
  int cached_ph = -1, ahead_ph = -1;                // phases held by that slot and by the other one (fetched ahead)
  volatile int* s_rec = reinterpret_cast<volatile int*>(ctrl + 768);
  const uint32_t s_rec_addr = smem_u32(ctrl + 768);
  int rec_ph = -1;                                  // thread 0: the phase whose record is (or is on its way) in s_rec
  const bool prof = (C.sched_flags & 2) != 0;        // per-phase and per-block time tables are kept (several %globaltimer reads and atomics per task)
  const SchedRec* prec = job_id == 0 ? C.train_rec : C.dec_rec;          // the same records inside the kernel parameter, when they fit
  const bool ptab = (job_id == 0 ? C.train_rec_n : C.dec_rec_n) > 0;
  auto need_rec = [&](int p) {                      // thread 0: make s_rec hold phase p's record
    if (rec_ph != p) {
#pragma unroll
      for (int q = 0; q < 4; q++) sched_cp16(s_rec_addr + 16 * q, reinterpret_cast<const char*>(J.rec + p) + 16 * q);
      rec_ph = p;
    }
    sched_cp_wait();
  };
  const int tid = threadIdx.x;
  u64 busy = 0;
  int rstep = -1, rph = -1;                         // thread 0: the (step, phase) last seen ready
  const unsigned total = (unsigned)J.nsteps * (unsigned)J.tasks_per_step;
  gemm_tc::GemmPipe gp; gp.stage_count[0] = gp.stage_count[1] = gp.tile_count[0] = gp.tile_count[1] = gp.tmem_base = 0;
  const bool use_tc = IsBf16<T>::value && job_id == 0;
  attn_tc::AttnPipe ap; ap.tasks = ap.stages = ap.stages2 = ap.a = ap.b = ap.done = 0;
  uint32_t bulk_uses = 0;                            // uses of the block's bulk-copy barrier (control area byte 104)
  uint32_t adam_tiles = 0;                           // tiles the block's AdamW tasks have staged (three barriers at control area byte 224)
  uint32_t ce_chunks = 0;                            // chunks the block's streamed cross-entropy tasks have staged (barriers at bytes 112, 120, 160, 168)
  if (use_tc) {
    if (tid == 0) {
      mbar_init(smem_u32(ctrl + 104), 1);
      for (int q = 0; q < ew::ADAM_STAGES; q++) mbar_init(smem_u32(ctrl + 224 + 8 * q), 1);
      for (int q = 0; q < 2; q++) { mbar_init(smem_u32(ctrl + 112 + 8 * q), 1); mbar_init(smem_u32(ctrl + 160 + 8 * q), 1); }   // streamed cross-entropy: four stages
    }
    attn_tc::block_init(ap, smem); gemm_tc::block_init(gp, smem, C.status);
  }
  // serving blocks: one mbarrier counts the bytes of the weight prefetch of the task they hold a ticket for
  const uint32_t fill_bar = smem_u32(ctrl + 96);
  uint32_t fills = 0;
  if (job_id == 1) {
    if (tid == 0) { mbar_init(fill_bar, 1); mbar_fence_init(); }
    dec::block_init<T, D, DH>(smem, C.md.T);
    __syncthreads();
  }
  u64 waited = 0, t_claim = 0, t_sync = 0, t_tail = 0, tl0 = 0, tl1 = 0;   // thread 0: where the time outside tasks goes
  bool c_any_rb = false;                             // thread 0: the phase last waited for has row-block dependencies (checked per task)
  int c_rb_off = -1, c_rb_map = 0;                   // thread 0: where and how the cached phase counts its completions per row block
  int c_ph = -1, c_lo = 0, c_hi = 0, c_mul = 0;      // thread 0: cached phase, its ticket range [c_lo, c_hi) within a step, and its test-only task permutation
  unsigned next_g = 0; bool have_next = false; unsigned claims = 0;   // thread 0: the ticket taken at the end of the previous task
  const bool early_ok = (C.sched_flags & 4) == 0;   // (flag 4: tickets only at the end of a task, for A/B measurements)
  for (;;) {
    if (tid == 0) {                                  // ---- claim (and, for the training job, wait for the dependencies)
      if (prof) { tl0 = gtimer(); if (tl1) t_tail += tl0 - tl1; }
      const u64 w_before = waited;
      int res = 0, step = 0, ph = 0, local = 0;
      // the abort / finished words are looked at inside every wait loop; here only now and then, a claim should not pay for them
      if ((claims++ & 15u) == 0 && (aborted(C.status) || (job_id == 1 && C.use_train && ld_relaxed(C.finished)))) res = -2;
      else {
        const unsigned g = have_next ? next_g : atomicAdd(J.ticket, 1u);
        have_next = false;
        if (g >= total) res = -2;
        else {
          step = (int)(g / (unsigned)J.tasks_per_step);
          const int r = (int)(g - (unsigned)step * (unsigned)J.tasks_per_step);
          // A block's tickets grow, so within a step it only moves forward through the phases: keep the current phase's
          // ticket range in registers and walk on, one scheduling record per phase passed. The record of the phase after
          // the one just worked on was requested at the end of the previous task and is normally already in shared memory.
          if (r < c_lo) { c_ph = -1; c_lo = 0; c_hi = 0; c_mul = 0; c_any_rb = false; }        // a new step
          if (ptab) {                                    // records in the kernel parameter: a walk over constant memory
            if (r >= c_hi) {
              int p = c_ph + 1;
              while (r >= prec[p].hi) p++;
              c_ph = p; c_lo = prec[p].lo; c_hi = prec[p].hi; c_mul = prec[p].perm_mul; c_rb_off = prec[p].rb_off; c_rb_map = prec[p].rb_map; c_any_rb = false;
            }
          } else {
            while (r >= c_hi) {
              c_ph++;
              need_rec(c_ph);
              c_lo = s_rec[0]; c_hi = s_rec[1]; c_mul = s_rec[3]; c_rb_off = s_rec[4]; c_rb_map = s_rec[5]; c_any_rb = false;
            }
          }
          ph = c_ph; local = r - c_lo;
          // test hook (SchedRec::perm_mul, 0 in production): tickets of a phase are handed out in a permuted task order, which
          // must not change any result - the reference's shuffled-order check (llm/gemm/test_gemm.cu:20-49)
          if (c_mul) local = (int)(((long long)local * c_mul + (c_mul >> 1)) % (long long)(c_hi - c_lo));
          // a phase whose dependencies are all phase-level stays ready once it has been seen ready; row-block dependencies are per task
          if (job_id == 0 && (!(step == rstep && ph == rph) || c_any_rb)) {
            const u64 w0 = prof ? gtimer() : 0;
            DepSet ds; int pro[4] = {0, 0, 0, 0};
            if (ptab) load_deps(ds, reinterpret_cast<const int*>(prec + ph)); else { need_rec(ph); load_deps(ds, s_rec); }
            if (ds.any_rb) {
#pragma unroll
              for (int k = 0; k < 4; k++) if (k < ds.cnt && ds.gr[k]) pro[k] = ptab ? prec[ds.ph[k]].rb_off : __ldg(&J.rec[ds.ph[k]].rb_off);
            }
            res = wait_deps(C, J, job_id, step, ph, local, ds, pro);
            c_any_rb = ds.any_rb;
            if (prof) {
              const u64 w = gtimer() - w0;
              waited += w;
              if (C.phase_busy && w > 200) atomicAdd(C.phase_busy + J.nph + ph, w);
            }
            if (res == 0) { rstep = step; rph = ph; }
          }
        }
      }
      s_sel[0] = res; s_sel[1] = step; s_sel[2] = ph; s_sel[3] = local; s_sel[5] = c_rb_off; s_sel[6] = c_rb_map;
      if (prof) { tl1 = gtimer(); t_claim += (tl1 - tl0) - (waited - w_before); }
    } else if (tid < 16) {
      sched_cp_wait();                               // the descriptor requested at the end of the last task: visible to all after the barrier below
    }
    __syncthreads();
    int res = s_sel[0];
    const int step = s_sel[1], ph = s_sel[2], local = s_sel[3];
    const int t_rb_off = s_sel[5], t_rb_map = s_sel[6];      // read now: thread 0 runs ahead of the thread that signals and rewrites these words for the next task
    if (res < 0) break;
    // The descriptor is read from shared memory: every dependency check ends with a device-scope acquire, after which L1 no
    // longer holds it, and the chain of dependent global loads that decoding it would take was a measurable part of the
    // per-task overhead. Two slots: the next phase's descriptor is requested at the end of a task (below), so a block that
    // moves on by one phase - the common case when phases have about as many tasks as there are blocks - finds it here.
    if (ph != cached_ph) {
      if (ph == ahead_ph) { slot ^= 1; ahead_ph = cached_ph; cached_ph = ph; }      // already there: no second barrier (-0.9 % per step)
      else {
        if (tid < (int)(sizeof(PhaseDesc) / 4)) reinterpret_cast<uint32_t*>(ctrl + 256 + 256 * slot)[tid] = __ldg(reinterpret_cast<const uint32_t*>(J.ph + ph) + tid);
        cached_ph = ph;
        __syncthreads();
      }
    }
    const PhaseDesc& d = *reinterpret_cast<const PhaseDesc*>(ctrl + 256 + 256 * slot);
    bool filled = false;
    if (job_id == 1) {                               // ---- serving: start the weight prefetch, THEN wait for the dependencies
      filled = dec::prefetch<T, D, DH>(C.dp, C.md, d.kind, d.i0, local, smem, fill_bar);
      if (tid == 0) {
        int r2 = 0;
        if (!(step == rstep && ph == rph)) {
          DepSet ds; int pro[4] = {0, 0, 0, 0};
          if (ptab) load_deps(ds, reinterpret_cast<const int*>(prec + ph)); else { need_rec(ph); load_deps(ds, s_rec); }
          r2 = wait_deps(C, J, job_id, step, ph, local, ds, pro);
          if (r2 == 0) { rstep = step; rph = ph; }
        }
        s_sel[4] = r2;
      }
      __syncthreads();
      res = s_sel[4];
      if (res < 0) {                                 // leaving with copies in flight: give them a bounded chance to land
        if (filled) mbar_wait(fill_bar, fills & 1u, C.status);
        __syncthreads();
        break;
      }
    }
    u64 t0 = 0;
    if (tid == 0) {
      if (prof) { t0 = gtimer(); t_sync += t0 - tl1; if (job_id == 1 && C.dp.trace && local == 0 && (ph == 0 || ph == 2)) C.dp.trace[16 + ph] = t0; }
    }
    if (job_id == 0) {
      // tensor-core tasks let their copy producer (this block's thread 0) take the next ticket as soon as its last copy is issued
      const EarlyTicket et = {(use_tc && early_ok) ? J.ticket : nullptr, s_sel + 7};
      if (tid == 0) s_sel[7] = 0;
      run_train_task<T, D, DH>(C, d, ph, local, step, smem, gp, ap, bulk_uses, adam_tiles, ce_chunks, et);
    }
    else run_decode_task<T, D, DH>(C, d, local, smem, fill_bar, fills & 1u);
    if (filled) fills++;
    __syncthreads();
    {                                                // ask for the next phase's descriptor and scheduling record now
      const int nxt = ph + 1 < J.nph ? ph + 1 : 0;
      if (nxt != ahead_ph) {
        if (tid >= 1 && tid <= (int)(sizeof(PhaseDesc) / 16))
          sched_cp16(smem_u32(ctrl + 256 + 256 * (slot ^ 1)) + 16 * (tid - 1), reinterpret_cast<const char*>(J.ph + nxt) + 16 * (tid - 1));
        ahead_ph = nxt;
      }
      if (tid == 0 && !ptab && rec_ph != nxt) {
#pragma unroll
        for (int q = 0; q < 4; q++) sched_cp16(s_rec_addr + 16 * q, reinterpret_cast<const char*>(J.rec + nxt) + 16 * q);
        rec_ph = nxt;
      }
    }
    // Two threads share the end of a task. Thread 0 takes the next ticket at once (a fetch-add whose value it needs only at the
    // top of the loop: the task is finished, so holding the next ticket cannot delay anything this block still has to do, every
    // dependency being a lower ticket). Thread 32 publishes the completion: ONE device-scope fence - the block barrier above
    // ordered every thread's writes of this task before it - and relaxed increments of the completion counters. The fence waits
    // for the SM's outstanding stores (about a microsecond after a GEMM epilogue); on its own thread it runs beside the ticket's
    // round trip and the next claim instead of in front of them.
    if (tid == 0) {
      if (job_id == 0 && s_sel[7] != 0) { next_g = (unsigned)s_sel[7] - 1u; have_next = true; }
      if (!have_next) { next_g = atomicAdd(J.ticket, 1u); have_next = true; }
      if (prof) {
        const u64 t1 = gtimer(); tl1 = t1;
        if (job_id == 1 && C.dp.trace && local == 0 && (ph == 0 || ph == 2)) C.dp.trace[17 + ph] = t1;
        busy += t1 - t0;
        if (job_id == 0 && C.phase_busy) {
          atomicAdd(C.phase_busy + ph, t1 - t0);
          if (step == C.prof_step) { atomicMin(C.phase_first + ph, t0); atomicMax(C.phase_last + ph, t1); }
        }
        if (job_id == 1 && C.dec_phase_busy) atomicAdd(C.dec_phase_busy + ph, t1 - t0);
      }
    } else if (tid == 32) {
      __threadfence();
      const int rb_off = t_rb_off, rb_map = t_rb_map;
      if (rb_off >= 0) {                               // completions per row block first: their waiters are the ones on the critical chain
        int prod, clo, chi; rb_of_task(rb_map, C.md, local, prod, clo, chi);
        red_relaxed_add(J.done_rb + rb_off + prod, 1);
      }
      if (ph != J.last_phase) red_relaxed_add(J.done + ph, 1);
      else {                                           // the step's last phase needs the old value
        const int old = atomicAdd(J.done + ph, 1);
        if (job_id == 0 && old == __ldg(J.ntasks + ph) * (step + 1) - 1) {     // last task of the step
          const u64 t1 = gtimer();
          C.step_done[step] = t1;
          if (C.live) C.live->steps = (unsigned)(step + 1);
          if (step == J.nsteps - 1) { *C.t_end = t1; __threadfence(); atomicExch(C.finished, 1); }
        }
      }
    }
  }
  sched_cp_wait();
  if (use_tc) gemm_tc::block_exit(gp, smem, C.status);
  if (tid == 0 && C.blk_busy) { C.blk_busy[blockIdx.x * 2 + job_id] = busy; if (job_id == 0 && C.blk_wait) { C.blk_wait[blockIdx.x] = waited; C.blk_wait[gridDim.x + blockIdx.x] = t_claim; C.blk_wait[2 * gridDim.x + blockIdx.x] = t_sync; C.blk_wait[3 * gridDim.x + blockIdx.x] = t_tail; } }
}

// A block of an idle partition must not leave before the whole grid has been placed: the hardware refills the slot of an
// exited block first, so early exits would steal the second block of the working SMs (measured: the 24-SM serving partition
// ran with one block per SM). Idle blocks therefore wait (bounded) until every block of the grid has reported in.
__device__ __forceinline__ void idle_block(const Ctx& C) {
  if (threadIdx.x == 0 && C.arrived) {
    const u64 t0 = gtimer();
    while (ld_relaxed(C.arrived) < (int)gridDim.x && gtimer() - t0 < 20000000ull) __nanosleep(500);
  }
}

template <class T, int D, int DH>
__global__ void __launch_bounds__(NTHR, 2) ofa_kernel(const __grid_constant__ Ctx C) {
  extern __shared__ __align__(1024) unsigned char dsm[];
  const unsigned hw = smid();
  const int rank = C.smid_rank ? C.smid_rank[hw] : (int)hw;
  const int isms = C.use_decode ? C.infer_sms : 0;
  if (threadIdx.x == 0 && C.arrived) atomicAdd(C.arrived, 1);
  const int role = rank < isms ? 1 : rank < isms + C.reserved_sms ? 2 : (rank < isms + C.reserved_sms + C.train_sms && C.use_train) ? 3 : 4;
  if (threadIdx.x == 0 && C.blk_info) C.blk_info[blockIdx.x] = (int)hw | (role << 16);
  if constexpr (IsBf16<T>::value) {
    // Blocks that never allocate TMEM give up their allocation permit at once. Measured on B200: while a resident block of a
    // kernel that contains tcgen05.alloc still holds the permit, the hardware does not place a second block of that kernel on
    // the SM; the serving partition ran with one block per SM (24 instead of 48 blocks) until this line was added.
    if (role != 3 && threadIdx.x < 32) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (role == 1) job_loop<T, D, DH>(C, C.dec, 1, dsm);
  else if (role == 3) job_loop<T, D, DH>(C, C.train, 0, dsm);
  else idle_block(C);
}

// one resident block per slot records its %smid so the host can build a dense rank table
__global__ void __launch_bounds__(NTHR, 2) smid_probe_kernel(unsigned* seen) {
  extern __shared__ __align__(1024) unsigned char dsm[];
  if (threadIdx.x == 0) {
    const unsigned id = smid();
    atomicOr(&seen[id >> 5], 1u << (id & 31));
    const u64 t0 = gtimer();
    while (gtimer() - t0 < 2000000ull) {}      // 2 ms: keeps the block resident so that every SM receives its share
    dsm[0] = 0;
  }
}

// first embedding of a decode context: xw := fx(wte[token] + wpe[pos])
template <class T, int D>
__global__ void decode_init_embed_kernel(DecodeParams P) { dec::write_embed<T, D>(P, P.st.scal[DS_TOKEN], P.st.scal[DS_POS]); }

}  // namespace ofa
