// Causal flash-attention for bf16 activations, head dim 64, on the 5th-generation tensor cores: forward, dK/dV and dQ tasks
// built from tcgen05.mma with accumulators in tensor memory, operands staged by TMA, and one softmax thread per row.
//
// Numerics follow the reference's tiles (llm/attention/attention.cuh:81-516): S = Q K^T in
// fp32, scaled by 0.125*log2(e), exponentiated in the exp2 domain with a running row maximum; P rounded to bf16 before P.V;
// O normalised in fp32 and rounded once; lse in natural log; backward recomputes P from lse, forms dS = P * (dP - D) in fp32,
// rounds P and dS to bf16 before the dV / dK / dQ products, and applies the 1/8 scale to dQ and dK at the end.
//
// Every task has the same three roles and the same step:
//   producer (warp 0, one thread)   TMA: the task's own 128-row tiles once, then per step two 64-row partner tiles
//   issuers  (warps 1 and 2, one thread each)   warp 1, group A: scores (and dP) of the step into tensor memory, as far
//                                   ahead of the softmax threads as the buffers allow;  warp 2, group B: the products that
//                                   consume what the softmax threads wrote to shared memory. Two threads because one thread
//                                   issues a tcgen05.mma only every ~96 cycles (measured) and because the two groups wait
//                                   for different things
//   softmax  (warps 4-7)            thread = row = tensor-memory lane: reads group A's result with tcgen05.ld, writes bf16
//                                   operands for group B into a SWIZZLE_128B K-major tile, hands both back with mbarriers
//   forward  step = 64 keys:    A: S = Q K_j^T            softmax: online max/sum, P_j        B: O += P_j V_j
//   dK/dV    step = 64 queries: A: S^T = K Q_i^T, dP^T = V dO_i^T      P^T, dS^T             B: dV += P^T dO_i, dK += dS^T Q_i
//   dQ       step = 64 keys:    A: S = Q K_j^T, dP = dO V_j^T          dS                    B: dQ += dS K_j
// Tensor memory (the block's 256 columns): forward S x2 at 0/64, O at 128; backward S 0, dP 64, accumulators 128, 192.
// Shared memory (the 96 KB pipeline area; the dK/dV task also keeps lse/D of its step in the staging area):
//   forward  Q 16 KB | 3 stages x (K_j, V_j) 16 KB | P x2 16 KB
//   dK/dV    K, V 32 KB | 2 stages x (Q_i, dO_i) 16 KB | P^T, dS^T 32 KB
//   dQ       Q, dO 32 KB | 3 stages x (K_j, V_j) 16 KB | dS 16 KB
// All waits are bounded (mbar_wait); a role that gives up leaves its loop and meets the others at the closing barrier.
#pragma once
#include <cuda.h>
#include "attn_common.cuh"
#include "gemm_tc.cuh"

namespace ofa {
namespace attn_tc {

using attn::DH; using attn::QTILE; using attn::KTILE; using attn::SCALE; using attn::SCALE_LOG2; using attn::LOG2E; using attn::LN2;

// barriers in the control area, from byte 832: q_full | st_full[3] | st_empty[3] | a_full[2] | a_free[2] | w_full[2] |
// b_full[2] | b_free[2] (reserved: no task waits on it since the forward output accumulates in tensor memory) | done |
// st2_full[2] | st2_empty[2] (the dK/dV task's two-stage ring)      (22 x 8 B)
constexpr int BAR0 = 832;
enum { B_QFULL = 0, B_STFULL = 1, B_STEMPTY = 4, B_AFULL = 7, B_AFREE = 9, B_WFULL = 11, B_BFULL = 13, B_BFREE = 15, B_DONE = 17, B_ST2FULL = 18, B_ST2EMPTY = 20, NBAR = 22 };
static_assert(BAR0 + 8 * NBAR <= CTRL_BYTES, "attention barriers do not fit the control area");
__device__ __forceinline__ uint32_t bar(uint32_t base, int i) { return base + gemm_tc::BAR_OFFSET + BAR0 + 8u * (uint32_t)i; }

// running counters (identical in every thread): tasks, stages loaded (three-stage ring, two-stage ring), steps (group A /
// softmax), forward PV tiles, backward tasks
struct AttnPipe { uint32_t tasks, stages, stages2, a, b, done; };

__device__ __forceinline__ void block_init(AttnPipe& ap, unsigned char* smem) {
  ap.tasks = ap.stages = ap.stages2 = ap.a = ap.b = ap.done = 0;
  if (threadIdx.x == 0) {
    const uint32_t base = smem_u32(smem);
    mbar_init(bar(base, B_QFULL), 1);
    for (int s = 0; s < 3; s++) { mbar_init(bar(base, B_STFULL + s), 1); mbar_init(bar(base, B_STEMPTY + s), 1); }
    for (int i = 0; i < 2; i++) {
      mbar_init(bar(base, B_AFULL + i), 1); mbar_init(bar(base, B_AFREE + i), 4); mbar_init(bar(base, B_WFULL + i), 4);
      mbar_init(bar(base, B_BFULL + i), 1); mbar_init(bar(base, B_BFREE + i), 4);
    }
    mbar_init(bar(base, B_DONE), 1);
    for (int s = 0; s < 2; s++) { mbar_init(bar(base, B_ST2FULL + s), 1); mbar_init(bar(base, B_ST2EMPTY + s), 1); }
    mbar_fence_init();
  }
}

// device-resident TMA descriptors of one layer's attention operands
struct Maps { CUtensorMap qkv128, qkv64, dO128, dO64; };   // boxes of 64 columns x 128 / 64 rows, SWIZZLE_128B

constexpr uint32_t IDESC_KK = umma_idesc(false, false, 128, 64);   // A and B K-major  (scores)
constexpr uint32_t IDESC_KM = umma_idesc(false, true, 128, 64);    // B MN-major       (products with a [k][64] tile)

// four k=16 steps of a 128 x 64 x 64 product; A K-major at sa, B K-major (b_mn = false) or MN-major at sb
__device__ __forceinline__ void mma_64(uint32_t d_tmem, uint32_t sa, uint32_t sb, bool b_mn, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < 4; kk++) {
    const u64 da = umma_smem_desc(sa + kk * 32, 16, 1024);
    const u64 db = b_mn ? umma_smem_desc(sb + kk * 2048, 8192, 1024) : umma_smem_desc(sb + kk * 32, 16, 1024);
    umma_bf16(d_tmem, da, db, b_mn ? IDESC_KM : IDESC_KK, (accumulate || kk > 0) ? 1u : 0u);
  }
}
__device__ __forceinline__ void bulk_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t b) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(b) : "memory");
}
__device__ __forceinline__ bool wait_or_abort(uint32_t b, uint32_t parity, DevStatus* st, int code, int phase_id, int task, int aux) {
  if (mbar_wait(b, parity, st)) return true;
  if (!aborted(st)) raise_abort(st, code, phase_id, task, aux);
  return false;
}
// a producer that gives up waits (bounded) for the copies it issued during this task that may still be in flight
__device__ __forceinline__ void drain(uint32_t base, int full0, uint32_t first, uint32_t next, uint32_t nstages) {
  for (uint32_t c = (next - first > nstages ? next - nstages : first); c < next; c++)
    for (int spin = 0; spin < 100000; spin++) if (mbar_try(bar(base, full0 + (int)(c % nstages)), (c / nstages) & 1)) break;
}
// one row's 32 consecutive bf16 pairs -> four 16-byte chunks (chunk0 .. chunk0+3) of a SWIZZLE_128B K-major tile row
__device__ __forceinline__ void store_chunks(unsigned char* tile, int row, int chunk0, const uint32_t (&pk)[16]) {
#pragma unroll
  for (int q = 0; q < 4; q++)
    *reinterpret_cast<uint4*>(tile + row * 128 + (((chunk0 + q) ^ (row & 7)) << 4)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// 2^x with the special-function unit's own instruction; results below 2^-126 flush to zero, which is what a probability that
// small rounds to in bf16 anyway
__device__ __forceinline__ float ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
// tcgen05.ld without the wait, so that several loads are in flight before tmem_ld_wait()
__device__ __forceinline__ void tmem_ld32_nw(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
                 "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
                 "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
                 "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
                 "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// softmax warps: release what they read / publish what they wrote (one arrival per warp)
__device__ __forceinline__ void warp_arrive(uint32_t b) { __syncwarp(); if ((threadIdx.x & 31) == 0) mbar_arrive(b); }

// ---------------------------------------------------------------------------------------------- forward
// Task (b, h, qt): 128 query rows q0 = qt*128; writes o[N, D] (bf16) and lse[B, H, T].
// The output row accumulates in tensor memory (PV_j adds to it). The running maximum a row's probabilities are taken
// against is only raised when the true maximum has grown by more than 2^8 since it was last set (probabilities then stay
// below 256, exact in fp32 sums and harmless in bf16), and only then is the accumulated row rescaled - read, multiplied and
// written back by its softmax thread between two products. Sum and output share the reference point, so the result is the
// same softmax; after the first tiles of a row the rescale is rare and the step is one pass over S.
constexpr float RESCALE_LOG2 = 8.f;
__device__ __noinline__ void fwd_task(const Maps* mp, bf16* o, float* lse, int b, int h, int qt, int T, int H, unsigned char* smem,
                                      AttnPipe& ap, uint32_t tmem, DevStatus* st, int phase_id, int task, const EarlyTicket& et) {
  const int D = H * DH;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t base = smem_u32(smem);
  const uint32_t sQ = base, sSt = base + 16384, sP = base + 65536;
  const int q0 = qt * QTILE, nrow0 = b * T;
  const int n = (q0 + QTILE) / KTILE;
  constexpr int NST = 3;
  if (warp == 0) {
    if (lane == 0) {                                                           // ---- producer
      fence_proxy_async();
      mbar_expect_tx(bar(base, B_QFULL), 16384);
      tma_load_2d(sQ, &mp->qkv128, bar(base, B_QFULL), h * DH, nrow0 + q0);
      uint32_t sc = ap.stages;
      for (int j = 0; j < n; j++, sc++) {
        const int s = sc % NST; const uint32_t use = sc / NST;
        if (!wait_or_abort(bar(base, B_STEMPTY + s), (use & 1) ^ 1, st, ST_MBAR_EMPTY_TIMEOUT, phase_id, task, j)) break;
        const uint32_t full = bar(base, B_STFULL + s);
        mbar_expect_tx(full, 16384);
        tma_load_2d(sSt + s * 16384, &mp->qkv64, full, D + h * DH, nrow0 + j * KTILE);
        tma_load_2d(sSt + s * 16384 + 8192, &mp->qkv64, full, 2 * D + h * DH, nrow0 + j * KTILE);
      }
      if (!aborted(st)) take_early_ticket(et);                               // the last copy of the task is on its way
      if (aborted(st)) drain(base, B_STFULL, ap.stages, sc, NST);
    }
  } else if (warp == 1) {
    if (lane == 0) {                                                           // ---- issuer of the scores: up to two steps ahead of the softmax threads
      bool ok = wait_or_abort(bar(base, B_QFULL), ap.tasks & 1, st, ST_MBAR_FULL_TIMEOUT, phase_id, task, 1000);
      for (int j = 0; j < n && ok; j++) {
        const uint32_t sc = ap.stages + j, c = ap.a + j; const int s = sc % NST;
        ok = wait_or_abort(bar(base, B_STFULL + s), (sc / NST) & 1, st, ST_MBAR_FULL_TIMEOUT, phase_id, task, j);
        if (ok && j >= 2) ok = wait_or_abort(bar(base, B_AFREE + (c & 1)), ((c - 2) >> 1) & 1, st, ST_MBAR_ACC_TIMEOUT, phase_id, task, j);
        if (!ok) break;
        tc_fence_after();
        mma_64(tmem + (c & 1) * 64, sQ, sSt + s * 16384, false, false);
        umma_commit(bar(base, B_AFULL + (c & 1)));
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {                                                           // ---- issuer of the products: follows the softmax threads
      bool ok = true;
      for (int i = 0; i < n && ok; i++) {                                      // O += P_i V_i
        const uint32_t sc = ap.stages + i, c = ap.a + i, cb = ap.b + i; const int s = sc % NST;
        ok = wait_or_abort(bar(base, B_WFULL + (c & 1)), (c >> 1) & 1, st, ST_MBAR_FULL_TIMEOUT, phase_id, task, 2000 + i);
        if (!ok) break;
        tc_fence_after();
        mma_64(tmem + 128, sP + (c & 1) * 16384, sSt + s * 16384 + 8192, true, i > 0);
        umma_commit(bar(base, B_STEMPTY + s));
        umma_commit(bar(base, B_BFULL + (cb & 1)));
      }
    }
  } else if (warp >= 4) {                                                      // ---- softmax threads: thread = query row
    const int e = warp - 4, r = e * 32 + lane, qg = q0 + r;
    const uint32_t tl = tmem + ((uint32_t)(e * 32) << 16);
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    auto wait_pv = [&](int i) {                                               // product i has been added to the output rows
      const uint32_t cb = ap.b + i;
      ok = mbar_wait(bar(base, B_BFULL + (cb & 1)), (cb >> 1) & 1, st);
      ok = __all_sync(0xffffffffu, ok);
    };
    for (int j = 0; j < n && ok; j++) {
      const uint32_t c = ap.a + j;
      const int k0 = j * KTILE;
      ok = mbar_wait(bar(base, B_AFULL + (c & 1)), (c >> 1) & 1, st);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      // Two passes over the 64 scores of the row, each reading them from tensor memory (a read costs far less than keeping 64
      // values live beside the packed probabilities: with both in registers the task spilled, and with the shared-memory
      // carve-out at its maximum a spill goes to L2): pass 1 finds the maximum, pass 2 exponentiates half a row at a time.
      const uint32_t ts = tl + (c & 1) * 64;
      const bool need_mask = __any_sync(0xffffffffu, k0 + KTILE - 1 > qg);       // warp-uniform: only tiles on the diagonal
      float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};             // four independent chains
      {
        uint32_t s0[32], s1[32];
        tmem_ld32_nw(ts, s0);
        tmem_ld32_nw(ts + 32, s1);
        tmem_ld_wait();
        if (!need_mask) {
#pragma unroll
          for (int x = 0; x < 32; x++) { mxa[x & 3] = fmaxf(mxa[x & 3], __uint_as_float(s0[x])); mxa[x & 3] = fmaxf(mxa[x & 3], __uint_as_float(s1[x])); }
        } else {
#pragma unroll
          for (int x = 0; x < 32; x++) {
            if (k0 + x <= qg) mxa[x & 3] = fmaxf(mxa[x & 3], __uint_as_float(s0[x]));   // masked scores contribute neither to the maximum nor to the sum
            if (k0 + 32 + x <= qg) mxa[x & 3] = fmaxf(mxa[x & 3], __uint_as_float(s1[x]));
          }
        }
      }
      const float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3]));
      const float m_true = fmaxf(m, mx * SCALE_LOG2);
      if (j == 0) m = m_true;                                                  // column 0 is visible to every row: finite
      else {
        const bool grow = m_true > m + RESCALE_LOG2;
        if (__any_sync(0xffffffffu, grow)) {                                   // rare after the first tiles: rescale this warp's rows
          wait_pv(j - 1);
          if (!ok) break;
          tc_fence_after();
          const float alpha = grow ? ex2(m - m_true) : 1.f;
          if (grow) { m = m_true; l *= alpha; }
#pragma unroll
          for (int hf = 0; hf < 2; hf++) {
            uint32_t rr[32];
            tmem_ld32(tl + 128 + hf * 32, rr);
#pragma unroll
            for (int x = 0; x < 32; x++) rr[x] = __float_as_uint(__uint_as_float(rr[x]) * alpha);
            tmem_st32(tl + 128 + hf * 32, rr);
          }
          tmem_st_wait();
          tc_fence_before();
        }
      }
      if (j >= 2) { wait_pv(j - 2); if (!ok) break; }                          // P buffer (c & 1) was last read by product j-2
      float rsa[4] = {0.f, 0.f, 0.f, 0.f};
      unsigned char* tile = smem + 65536 + (c & 1) * 16384;
      const float nm = -m;
#pragma unroll
      for (int hf = 0; hf < 2; hf++) {
        uint32_t sv[32], pk[16];
        tmem_ld32_nw(ts + hf * 32, sv);
        tmem_ld_wait();
        if (hf == 1) { tc_fence_before(); warp_arrive(bar(base, B_AFREE + (c & 1))); }   // S_j has been read for the last time
        if (need_mask) {
#pragma unroll
          for (int x = 0; x < 32; x++) if (k0 + hf * 32 + x > qg) sv[x] = 0xff800000u;   // -inf: 2^-inf = 0
        }
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          const float p0 = ex2(fmaf(__uint_as_float(sv[x]), SCALE_LOG2, nm)), p1 = ex2(fmaf(__uint_as_float(sv[x + 1]), SCALE_LOG2, nm));
          rsa[(x >> 1) & 3] += p0 + p1;
          pk[x >> 1] = pack2(p0, p1);
        }
        store_chunks(tile, r, hf * 4, pk);
      }
      const float rs = (rsa[0] + rsa[1]) + (rsa[2] + rsa[3]);
      l += rs;
      fence_async_smem();
      warp_arrive(bar(base, B_WFULL + (c & 1)));
    }
    if (ok && n >= 2) wait_pv(n - 2);
    if (ok) wait_pv(n - 1);
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l;
      bf16* dst = o + (size_t)(nrow0 + qg) * D + h * DH;
#pragma unroll
      for (int hf = 0; hf < 2; hf++) {
        uint32_t rr[32];
        tmem_ld32(tl + 128 + hf * 32, rr);
#pragma unroll
        for (int q = 0; q < 4; q++) {
          uint4 v;
          v.x = pack2(__uint_as_float(rr[8 * q]) * inv, __uint_as_float(rr[8 * q + 1]) * inv); v.y = pack2(__uint_as_float(rr[8 * q + 2]) * inv, __uint_as_float(rr[8 * q + 3]) * inv);
          v.z = pack2(__uint_as_float(rr[8 * q + 4]) * inv, __uint_as_float(rr[8 * q + 5]) * inv); v.w = pack2(__uint_as_float(rr[8 * q + 6]) * inv, __uint_as_float(rr[8 * q + 7]) * inv);
          *reinterpret_cast<uint4*>(dst + hf * 32 + 8 * q) = v;
        }
      }
      lse[((size_t)b * H + h) * T + qg] = m * LN2 + logf(l);
    }
  }
  ap.tasks += 1; ap.stages += (uint32_t)n; ap.a += (uint32_t)n; ap.b += (uint32_t)n;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
}

// ---------------------------------------------------------------------------------------------- backward: dK, dV
// Task (b, h, kt): 128 key rows k0 = kt*128; walks query blocks of 64 rows from the diagonal to the end of the sequence.
__device__ __noinline__ void bwd_dkdv_task(const Maps* mp, const float* lse, const float* Dr, bf16* dqkv, int b, int h, int kt, int T, int H,
                                           unsigned char* smem, AttnPipe& ap, uint32_t tmem, DevStatus* st, int phase_id, int task, const EarlyTicket& et) {
  const int D = H * DH, ld = 3 * D;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t base = smem_u32(smem);
  const uint32_t sK = base, sV = base + 16384, sSt = base + 32768, sPT = base + 65536, sDT = base + 81920;
  const uint32_t sStat = base + gemm_tc::PIPE_BYTES;            // stage s: lse at +s*512, D at +s*512+256
  const int k0 = kt * QTILE, nrow0 = b * T;
  const int i0 = k0 / KTILE, n = T / KTILE - i0;
  constexpr int NST = 2;
  const uint32_t st0 = ap.stages2;                              // this task's ring has its own barriers and counter
  if (warp == 0) {
    if (lane == 0) {                                                           // ---- producer
      fence_proxy_async();
      mbar_expect_tx(bar(base, B_QFULL), 32768);
      tma_load_2d(sK, &mp->qkv128, bar(base, B_QFULL), D + h * DH, nrow0 + k0);
      tma_load_2d(sV, &mp->qkv128, bar(base, B_QFULL), 2 * D + h * DH, nrow0 + k0);
      const float* Lg = lse + ((size_t)b * H + h) * T; const float* Dg = Dr + ((size_t)b * H + h) * T;
      uint32_t sc = st0;
      for (int i = 0; i < n; i++, sc++) {
        const int s = sc % NST; const uint32_t use = sc / NST;
        if (!wait_or_abort(bar(base, B_ST2EMPTY + s), (use & 1) ^ 1, st, ST_MBAR_EMPTY_TIMEOUT, phase_id, task, i)) break;
        const uint32_t full = bar(base, B_ST2FULL + s);
        mbar_expect_tx(full, 16384 + 512);
        tma_load_2d(sSt + s * 16384, &mp->qkv64, full, h * DH, nrow0 + (i0 + i) * KTILE);
        tma_load_2d(sSt + s * 16384 + 8192, &mp->dO64, full, h * DH, nrow0 + (i0 + i) * KTILE);
        bulk_1d(sStat + s * 512, Lg + (i0 + i) * KTILE, 256, full);
        bulk_1d(sStat + s * 512 + 256, Dg + (i0 + i) * KTILE, 256, full);
      }
      if (!aborted(st)) take_early_ticket(et);
      if (aborted(st)) drain(base, B_ST2FULL, st0, sc, NST);
    }
  } else if (warp == 1) {
    if (lane == 0) {                                                           // ---- issuer of the scores: runs one step ahead of the softmax threads
      bool ok = wait_or_abort(bar(base, B_QFULL), ap.tasks & 1, st, ST_MBAR_FULL_TIMEOUT, phase_id, task, 1000);
      for (int i = 0; i < n && ok; i++) {
        const uint32_t sc = st0 + i, c = ap.a + i; const int s = sc % NST;
        ok = wait_or_abort(bar(base, B_ST2FULL + s), (sc / NST) & 1, st, ST_MBAR_FULL_TIMEOUT, phase_id, task, i);
        if (ok && i >= 1) ok = wait_or_abort(bar(base, B_AFREE + ((c - 1) & 1)), ((c - 1) >> 1) & 1, st, ST_MBAR_ACC_TIMEOUT, phase_id, task, i);
        if (!ok) break;
        tc_fence_after();
        mma_64(tmem, sK, sSt + s * 16384, false, false);                       // S^T  = K Q_i^T
        mma_64(tmem + 64, sV, sSt + s * 16384 + 8192, false, false);           // dP^T = V dO_i^T
        umma_commit(bar(base, B_AFULL + (c & 1)));
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {                                                           // ---- issuer of the products: follows the softmax threads
      bool ok = true;
      for (int i = 0; i < n && ok; i++) {
        const uint32_t sc = st0 + i, c = ap.a + i; const int s = sc % NST;
        ok = wait_or_abort(bar(base, B_WFULL + (c & 1)), (c >> 1) & 1, st, ST_MBAR_FULL_TIMEOUT, phase_id, task, 2000 + i);
        if (!ok) break;
        tc_fence_after();
        mma_64(tmem + 128, sPT, sSt + s * 16384 + 8192, true, i > 0);          // dV += P^T dO_i
        mma_64(tmem + 192, sDT, sSt + s * 16384, true, i > 0);                 // dK += dS^T Q_i
        umma_commit(bar(base, B_ST2EMPTY + s));
        if (i == n - 1) umma_commit(bar(base, B_DONE));
      }
    }
  } else if (warp >= 4) {                                                      // ---- softmax threads: thread = key row
    const int e = warp - 4, r = e * 32 + lane, kg = k0 + r;
    const uint32_t tl = tmem + ((uint32_t)(e * 32) << 16);
    bool ok = true;
    for (int i = 0; i < n && ok; i++) {
      const uint32_t sc = st0 + i, c = ap.a + i; const int s = sc % NST;
      const int qi0 = (i0 + i) * KTILE;
      ok = mbar_wait(bar(base, B_ST2FULL + s), (sc / NST) & 1, st) && mbar_wait(bar(base, B_AFULL + (c & 1)), (c >> 1) & 1, st);   // lse, D of the stage; S^T, dP^T
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const float* sL = reinterpret_cast<const float*>(smem + gemm_tc::PIPE_BYTES + s * 512); const float* sD = sL + 64;
      const bool need_mask = __any_sync(0xffffffffu, qi0 < kg);                 // warp-uniform: only blocks on the diagonal
      uint32_t pp[2][16], pd[2][16];
#pragma unroll
      for (int hf = 0; hf < 2; hf++) {
        uint32_t rs[32], rd[32];
        tmem_ld32_nw(tl + hf * 32, rs);
        tmem_ld32_nw(tl + 64 + hf * 32, rd);
        tmem_ld_wait();
        if (hf == 1) {                                                         // everything of this step is in registers: the next scores may overwrite it
          tc_fence_before();
          warp_arrive(bar(base, B_AFREE + (c & 1)));
        }
        if (need_mask) {                                                       // a masked score becomes -inf: 2^-inf = 0 for P, and dS = 0 * (..) = 0
#pragma unroll
          for (int x = 0; x < 32; x++) if (kg > qi0 + hf * 32 + x) rs[x] = 0xff800000u;
        }
#pragma unroll
        for (int x = 0; x < 32; x += 4) {                                      // the step's lse and D: four queries per 16-byte read
          const float4 l4 = reinterpret_cast<const float4*>(sL)[(hf * 32 + x) >> 2], d4 = reinterpret_cast<const float4*>(sD)[(hf * 32 + x) >> 2];
          const float p0 = ex2(fmaf(__uint_as_float(rs[x]), SCALE_LOG2, -l4.x * LOG2E)), p1 = ex2(fmaf(__uint_as_float(rs[x + 1]), SCALE_LOG2, -l4.y * LOG2E));
          const float p2 = ex2(fmaf(__uint_as_float(rs[x + 2]), SCALE_LOG2, -l4.z * LOG2E)), p3 = ex2(fmaf(__uint_as_float(rs[x + 3]), SCALE_LOG2, -l4.w * LOG2E));
          const float d0 = p0 * (__uint_as_float(rd[x]) - d4.x), d1 = p1 * (__uint_as_float(rd[x + 1]) - d4.y);
          const float d2 = p2 * (__uint_as_float(rd[x + 2]) - d4.z), d3 = p3 * (__uint_as_float(rd[x + 3]) - d4.w);
          pp[hf][x >> 1] = pack2(p0, p1); pd[hf][x >> 1] = pack2(d0, d1);
          pp[hf][(x >> 1) + 1] = pack2(p2, p3); pd[hf][(x >> 1) + 1] = pack2(d2, d3);
        }
      }
      if (i >= 1) {                                                            // the previous step's products read the tiles about to be rewritten
        const uint32_t scp = sc - 1;
        ok = mbar_wait(bar(base, B_ST2EMPTY + (int)(scp % NST)), (scp / NST) & 1, st);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
#pragma unroll
      for (int hf = 0; hf < 2; hf++) { store_chunks(smem + 65536, r, hf * 4, pp[hf]); store_chunks(smem + 81920, r, hf * 4, pd[hf]); }
      fence_async_smem();
      warp_arrive(bar(base, B_WFULL + (c & 1)));
    }
    if (ok) { ok = mbar_wait(bar(base, B_DONE), ap.done & 1, st); ok = __all_sync(0xffffffffu, ok); }
    if (ok) {
      tc_fence_after();
#pragma unroll
      for (int which = 0; which < 2; which++) {                                // 0: dV, 1: dK (scaled)
        const float sc = which ? SCALE : 1.f;
        bf16* dst = dqkv + (size_t)(nrow0 + kg) * ld + (which ? D : 2 * D) + h * DH;
#pragma unroll
        for (int hf = 0; hf < 2; hf++) {
          uint32_t rr[32];
          tmem_ld32(tl + 128 + which * 64 + hf * 32, rr);
#pragma unroll
          for (int q = 0; q < 4; q++) {
            uint4 v;
            v.x = pack2(__uint_as_float(rr[8 * q]) * sc, __uint_as_float(rr[8 * q + 1]) * sc); v.y = pack2(__uint_as_float(rr[8 * q + 2]) * sc, __uint_as_float(rr[8 * q + 3]) * sc);
            v.z = pack2(__uint_as_float(rr[8 * q + 4]) * sc, __uint_as_float(rr[8 * q + 5]) * sc); v.w = pack2(__uint_as_float(rr[8 * q + 6]) * sc, __uint_as_float(rr[8 * q + 7]) * sc);
            *reinterpret_cast<uint4*>(dst + hf * 32 + 8 * q) = v;
          }
        }
      }
    }
  }
  ap.tasks += 1; ap.stages2 += (uint32_t)n; ap.a += (uint32_t)n; ap.done += 1;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
}

// ---------------------------------------------------------------------------------------------- backward: dQ
// Task (b, h, qt): 128 query rows; walks key blocks of 64 rows from 0 to the diagonal.
__device__ __noinline__ void bwd_dq_task(const Maps* mp, const float* lse, const float* Dr, bf16* dqkv, int b, int h, int qt, int T, int H,
                                         unsigned char* smem, AttnPipe& ap, uint32_t tmem, DevStatus* st, int phase_id, int task, const EarlyTicket& et) {
  const int D = H * DH, ld = 3 * D;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t base = smem_u32(smem);
  const uint32_t sQ = base, sdO = base + 16384, sSt = base + 32768, sDS = base + 81920;
  const int q0 = qt * QTILE, nrow0 = b * T;
  const int n = (q0 + QTILE) / KTILE;
  constexpr int NST = 3;
  if (warp == 0) {
    if (lane == 0) {                                                           // ---- producer
      fence_proxy_async();
      mbar_expect_tx(bar(base, B_QFULL), 32768);
      tma_load_2d(sQ, &mp->qkv128, bar(base, B_QFULL), h * DH, nrow0 + q0);
      tma_load_2d(sdO, &mp->dO128, bar(base, B_QFULL), h * DH, nrow0 + q0);
      uint32_t sc = ap.stages;
      for (int j = 0; j < n; j++, sc++) {
        const int s = sc % NST; const uint32_t use = sc / NST;
        if (!wait_or_abort(bar(base, B_STEMPTY + s), (use & 1) ^ 1, st, ST_MBAR_EMPTY_TIMEOUT, phase_id, task, j)) break;
        const uint32_t full = bar(base, B_STFULL + s);
        mbar_expect_tx(full, 16384);
        tma_load_2d(sSt + s * 16384, &mp->qkv64, full, D + h * DH, nrow0 + j * KTILE);
        tma_load_2d(sSt + s * 16384 + 8192, &mp->qkv64, full, 2 * D + h * DH, nrow0 + j * KTILE);
      }
      if (!aborted(st)) take_early_ticket(et);                               // the last copy of the task is on its way
      if (aborted(st)) drain(base, B_STFULL, ap.stages, sc, NST);
    }
  } else if (warp == 1) {
    if (lane == 0) {                                                           // ---- issuer of the scores: runs one step ahead of the softmax threads
      bool ok = wait_or_abort(bar(base, B_QFULL), ap.tasks & 1, st, ST_MBAR_FULL_TIMEOUT, phase_id, task, 1000);
      for (int j = 0; j < n && ok; j++) {
        const uint32_t sc = ap.stages + j, c = ap.a + j; const int s = sc % NST;
        ok = wait_or_abort(bar(base, B_STFULL + s), (sc / NST) & 1, st, ST_MBAR_FULL_TIMEOUT, phase_id, task, j);
        if (ok && j >= 1) ok = wait_or_abort(bar(base, B_AFREE + ((c - 1) & 1)), ((c - 1) >> 1) & 1, st, ST_MBAR_ACC_TIMEOUT, phase_id, task, j);
        if (!ok) break;
        tc_fence_after();
        mma_64(tmem, sQ, sSt + s * 16384, false, false);                       // S  = Q K_j^T
        mma_64(tmem + 64, sdO, sSt + s * 16384 + 8192, false, false);          // dP = dO V_j^T
        umma_commit(bar(base, B_AFULL + (c & 1)));
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {                                                           // ---- issuer of the products: follows the softmax threads
      bool ok = true;
      for (int j = 0; j < n && ok; j++) {
        const uint32_t sc = ap.stages + j, c = ap.a + j; const int s = sc % NST;
        ok = wait_or_abort(bar(base, B_WFULL + (c & 1)), (c >> 1) & 1, st, ST_MBAR_FULL_TIMEOUT, phase_id, task, 2000 + j);
        if (!ok) break;
        tc_fence_after();
        mma_64(tmem + 128, sDS, sSt + s * 16384, true, j > 0);                 // dQ += dS K_j
        umma_commit(bar(base, B_STEMPTY + s));
        if (j == n - 1) umma_commit(bar(base, B_DONE));
      }
    }
  } else if (warp >= 4) {                                                      // ---- softmax threads: thread = query row
    const int e = warp - 4, r = e * 32 + lane, qg = q0 + r;
    const uint32_t tl = tmem + ((uint32_t)(e * 32) << 16);
    const float lse2 = lse[((size_t)b * H + h) * T + qg] * LOG2E, dr = Dr[((size_t)b * H + h) * T + qg];
    bool ok = true;
    for (int j = 0; j < n && ok; j++) {
      const uint32_t c = ap.a + j;
      const int k0 = j * KTILE;
      ok = mbar_wait(bar(base, B_AFULL + (c & 1)), (c >> 1) & 1, st);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool need_mask = __any_sync(0xffffffffu, k0 + KTILE - 1 > qg);      // warp-uniform: only blocks on the diagonal
      uint32_t pd[2][16];
#pragma unroll
      for (int hf = 0; hf < 2; hf++) {
        uint32_t rs[32], rd[32];
        tmem_ld32_nw(tl + hf * 32, rs);
        tmem_ld32_nw(tl + 64 + hf * 32, rd);
        tmem_ld_wait();
        if (hf == 1) {                                                         // everything of this step is in registers: the next scores may overwrite it
          tc_fence_before();
          warp_arrive(bar(base, B_AFREE + (c & 1)));
        }
        if (need_mask) {
#pragma unroll
          for (int x = 0; x < 32; x++) if (k0 + hf * 32 + x > qg) rs[x] = 0xff800000u;
        }
#pragma unroll
        for (int x = 0; x < 32; x += 2) {
          const float p0 = ex2(fmaf(__uint_as_float(rs[x]), SCALE_LOG2, -lse2)), p1 = ex2(fmaf(__uint_as_float(rs[x + 1]), SCALE_LOG2, -lse2));
          pd[hf][x >> 1] = pack2(p0 * (__uint_as_float(rd[x]) - dr), p1 * (__uint_as_float(rd[x + 1]) - dr));
        }
      }
      if (j >= 1) {                                                            // the previous step's product read the tile about to be rewritten
        const uint32_t scp = ap.stages + j - 1;
        ok = mbar_wait(bar(base, B_STEMPTY + (int)(scp % NST)), (scp / NST) & 1, st);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      store_chunks(smem + 81920, r, 0, pd[0]);
      store_chunks(smem + 81920, r, 4, pd[1]);
      fence_async_smem();
      warp_arrive(bar(base, B_WFULL + (c & 1)));
    }
    if (ok) { ok = mbar_wait(bar(base, B_DONE), ap.done & 1, st); ok = __all_sync(0xffffffffu, ok); }
    if (ok) {
      tc_fence_after();
      bf16* dst = dqkv + (size_t)(nrow0 + qg) * ld + h * DH;
#pragma unroll
      for (int hf = 0; hf < 2; hf++) {
        uint32_t rr[32];
        tmem_ld32(tl + 128 + hf * 32, rr);
#pragma unroll
        for (int q = 0; q < 4; q++) {
          uint4 v;
          v.x = pack2(__uint_as_float(rr[8 * q]) * SCALE, __uint_as_float(rr[8 * q + 1]) * SCALE); v.y = pack2(__uint_as_float(rr[8 * q + 2]) * SCALE, __uint_as_float(rr[8 * q + 3]) * SCALE);
          v.z = pack2(__uint_as_float(rr[8 * q + 4]) * SCALE, __uint_as_float(rr[8 * q + 5]) * SCALE); v.w = pack2(__uint_as_float(rr[8 * q + 6]) * SCALE, __uint_as_float(rr[8 * q + 7]) * SCALE);
          *reinterpret_cast<uint4*>(dst + hf * 32 + 8 * q) = v;
        }
      }
    }
  }
  ap.tasks += 1; ap.stages += (uint32_t)n; ap.a += (uint32_t)n; ap.done += 1;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
}

}  // namespace attn_tc
}  // namespace ofa
