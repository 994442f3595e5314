// Device-side building blocks shared by every task of the megakernel: PTX wrappers for the sm_100a asynchronous
// machinery (mbarrier, TMA, tcgen05/TMEM), bounded waits, the abort/status protocol, and small math helpers.
//
// Conventions used by all task code:
//   * a task is executed by ALL 256 threads of one block (`ofa::NTHR`), never looks at blockIdx/gridDim, and ends with a
//     block-wide barrier so the caller may reuse shared memory;
//   * no wait in this library is unbounded: every spin has a %globaltimer deadline and also watches the global abort
//     word; a wait that gives up records {code, phase, task, block} once and raises the abort word so that every
//     other waiter in the grid drains and the kernel returns instead of hanging the GPU.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>

namespace ofa {

typedef __nv_bfloat16 bf16;
typedef unsigned long long u64;
constexpr int NTHR = 256;   // threads per block (task contract)

// ---------------------------------------------------------------------------------------------- status / abort
enum StatusCode : int {
  ST_OK = 0,
  ST_DEP_TIMEOUT = 1,       // a dependency counter did not reach its target in time
  ST_MBAR_FULL_TIMEOUT = 2, // TMA bytes never arrived
  ST_MBAR_EMPTY_TIMEOUT = 3,// MMA never released a pipeline stage
  ST_MBAR_ACC_TIMEOUT = 4,  // accumulator hand-off (MMA <-> epilogue) never happened
  ST_SMEM_MISALIGNED = 5,
  ST_EXTERNAL_TIMEOUT = 6,  // a flag owned by the host / another rank was not raised in time
  ST_BAD_DESC = 7,
};
struct DevStatus {          // lives in device global memory, zero-initialised by the host
  int code;                 // first failure wins (atomicCAS from 0)
  int phase, task, block, aux;
  int abort;                // != 0: every spin in the grid gives up
};

__device__ __forceinline__ u64 gtimer() { u64 t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ unsigned smid() { unsigned r; asm volatile("mov.u32 %0, %%smid;" : "=r"(r)); return r; }
__device__ __forceinline__ int ld_acquire(const int* p) { int v; asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ int ld_relaxed(const int* p) { int v; asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ void fence_acquire() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
__device__ __forceinline__ void red_relaxed_add(int* p, int v) { asm volatile("red.relaxed.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void red_release_add(int* p, int v) { asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }

__device__ __forceinline__ void raise_abort(DevStatus* st, int code, int phase, int task, int aux) {
  if (atomicCAS(&st->code, 0, code) == 0) { st->phase = phase; st->task = task; st->block = (int)blockIdx.x; st->aux = aux; }
  __threadfence();
  atomicExch(&st->abort, 1);
}
__device__ __forceinline__ bool aborted(const DevStatus* st) { return ld_relaxed(&st->abort) != 0; }

// ---------------------------------------------------------------------------------------------- small math
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block reductions over 256 threads; `red` = 8 floats of shared scratch; result valid in all threads; fixed order.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int i = 1; i < NTHR / 32; i++) r += red[i];
  return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int i = 1; i < NTHR / 32; i++) r = fmaxf(r, red[i]);
  return r;
}

// storage-type helpers: the same task code runs on bf16 (GPT-S) and fp32 (tiny model) activations
template <class T> struct Vec;   // 16-byte vector of T
template <> struct Vec<bf16> { static constexpr int N = 8; };
template <> struct Vec<float> { static constexpr int N = 4; };
__device__ __forceinline__ float to_f(bf16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_f(float x) { return x; }
template <class T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ bf16 from_f<bf16>(float x) { return __float2bfloat16(x); }
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
// value after a round trip through the storage type (identity for fp32)
template <class T> __device__ __forceinline__ float round_to(float x) { return to_f(from_f<T>(x)); }

__device__ __forceinline__ void unpack8(uint4 u, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) { float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}
__device__ __forceinline__ uint32_t pack2f(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// load / store `Vec<T>::N` consecutive elements (16 bytes) as floats
__device__ __forceinline__ void ldv(const bf16* p, float* f) { unpack8(*reinterpret_cast<const uint4*>(p), f); }
__device__ __forceinline__ void ldv(const float* p, float* f) { float4 v = *reinterpret_cast<const float4*>(p); f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
__device__ __forceinline__ void stv(bf16* p, const float* f) { *reinterpret_cast<uint4*>(p) = pack8(f); }
__device__ __forceinline__ void stv(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }

// GELU (tanh form) and its derivative. FAST selects tanh.approx.f32 (bf16 training path); otherwise tanhf.
template <bool FAST> __device__ __forceinline__ float tanh_sel(float x) {
  if constexpr (FAST) { float y; asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
  else return tanhf(x);
}
template <bool FAST> __device__ __forceinline__ float gelu_fwd(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanh_sel<FAST>(u));
}
template <bool FAST> __device__ __forceinline__ float gelu_bwd(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  const float t = tanh_sel<FAST>(u);
  const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
}

// 2^x on the special-function unit (results below 2^-126 flush to zero; 2^-inf = 0)
__device__ __forceinline__ float ex2_approx(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

__device__ __forceinline__ u64 splitmix64(u64 z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// ---------------------------------------------------------------------------------------------- sm_100a async machinery
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: true when the phase with `parity` completed; false when the deadline passed or the grid is aborting.
// The common case - the phase is already complete or completes within the first probe - must stay a handful of
// instructions in the caller: with the polling loops inlined, a wait on a completed barrier measured 174 cycles instead of
// the 14 of one mbarrier.try_wait, on every pipeline stage of every tile.
constexpr u64 MBAR_TIMEOUT_NS = 2000000000ull;   // 2 s: far beyond any legitimate wait inside one tile
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, const DevStatus* st) {
#pragma unroll 1
  for (int i = 0; i < 128; i++) if (mbar_try(bar, parity)) return true;
  const u64 t0 = gtimer();
#pragma unroll 1
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; i++) if (mbar_try(bar, parity)) return true;
    if (st && aborted(st)) return false;
    if (gtimer() - t0 > MBAR_TIMEOUT_NS) return false;
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const DevStatus* st) {
  if (mbar_try(bar, parity)) return true;
  if (mbar_try(bar, parity)) return true;      // a try_wait blocks for a while by itself: the second probe catches most short waits
  return mbar_wait_slow(bar, parity, st);
}

// The next ticket of the block's job, taken by thread 0 from inside a task once its own part of the task is over (the copy
// producer after its last copy): the fetch-add's round trip then runs beside the rest of the task instead of after it.
// slot: a word of the control area, 0 = nothing taken, else ticket + 1. counter == nullptr: not offered (serving job).
struct EarlyTicket { unsigned* counter; volatile int* slot; };
__device__ __forceinline__ void take_early_ticket(const EarlyTicket& e) { if (e.counter) *e.slot = (int)(atomicAdd(e.counter, 1u) + 1u); }

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
// 2-D tiled TMA load (no multicast), completion counted in bytes on `bar`. c0 = innermost coordinate (elements).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t ncols) {   // one full warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {      // one full warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate; issued by ONE thread.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, u64 desc_a, u64 desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
// arrive on `bar` once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 TMEM lanes (this warp's quadrant) x 32 fp32 columns -> 32 registers per thread (thread = lane = row)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
                 "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
                 "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
               : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory operand descriptor for tcgen05.mma, SWIZZLE_128B canonical layouts (descriptor version 1):
//   bits [0,14) start address >> 4, [16,30) leading-dimension byte offset >> 4, [32,46) stride byte offset >> 4,
//   bit 46 version, bits [61,64) swizzle mode (2 = 128 B).
__device__ __forceinline__ u64 umma_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (u64)((saddr & 0x3FFFFu) >> 4) | ((u64)(lbo_bytes >> 4) << 16) | ((u64)(sbo_bytes >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: D fp32 (bit 4), A/B bf16 (bits 7, 10), operand majorness (bits 15/16: 1 = MN-major),
// N>>3 at bit 17, M>>4 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc(bool a_mn_major, bool b_mn_major, int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

}  // namespace ofa
