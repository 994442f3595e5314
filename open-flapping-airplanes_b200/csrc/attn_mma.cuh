// Causal flash-attention for bf16 activations, head dim 64: forward, backward-prep, dK/dV and dQ tasks, staged through
// swizzled shared memory with cp.async double buffering and mma.sync.m16n8k16 (fp32 accumulate).
//
// Numerics follow the reference tiles (llm/attention/attention.cuh:81-516): S = Q K^T in fp32, scaled by 0.125*log2(e) and
// exponentiated in the exp2 domain with a running row maximum; P is rounded to bf16 before P.V; O is normalised in fp32 and
// rounded once; lse is stored in natural log; backward recomputes P from lse, forms dS = P * (dP - D) in fp32 and rounds P
// and dS to bf16 before the dV / dK / dQ products; the 1/8 scale is applied to dQ and dK at the end.
// The decomposition differs from the reference: a task covers 128 rows (one 16-row slab per warp, so no cross-warp merge
// of partial softmax state is needed), and the backward tasks walk their 64-row partner tiles in two 32-wide halves to
// stay inside 128 registers.
//
// Layouts: qkv [N, 3D] (q | k | v, head h at columns h*64), o [N, D], lse/Dr [B, H, T] fp32, dqkv [N, 3D] (dq | dk | dv).
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

constexpr int SMEM_FWD = QTILE * 128 + 2 * 2 * KTILE * 128;                  // Q + 2 x (K, V)            = 49,152 B
constexpr int SMEM_DKDV = 2 * QTILE * 128 + 2 * 2 * KTILE * 128 + 2 * 2 * KTILE * 4;   // K,V + 2x(Q,dO) + 2x(lse,D) = 66,560 B
constexpr int SMEM_DQ = 2 * QTILE * 128 + 2 * 2 * KTILE * 128;               // Q,dO + 2 x (K, V)         = 65,536 B

// ---------------------------------------------------------------------------------------------- primitives
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// A tile row is 64 bf16 = 128 B = eight 16-byte chunks; chunk c of row r is stored at position c ^ (r & 7).
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) { return base + row * 128 + ((chunk ^ (row & 7)) << 4); }

// rows [row0, row0+nrows) x 64 columns starting at `col0` of a [*, ld] bf16 matrix -> swizzled tile (all 256 threads)
__device__ __forceinline__ void load_tile(uint32_t sbase, const bf16* g, int ld, int row0, int col0, int nrows) {
  for (int i = threadIdx.x; i < nrows * 8; i += NTHR) {
    const int r = i >> 3, c = i & 7;
    cp_async16(tile_addr(sbase, r, c), g + (size_t)(row0 + r) * ld + col0 + c * 8);
  }
}
// A fragment (16 rows x 16 k) of a swizzled tile: rows row0.., k chunk pair ks (columns ks*16..ks*16+15)
__device__ __forceinline__ void load_a(uint32_t sbase, int row0, int ks, uint32_t (&a)[4]) {
  const int lane = threadIdx.x & 31;
  ldsm4(tile_addr(sbase, row0 + (lane & 15), ks * 2 + (lane >> 4)), a[0], a[1], a[2], a[3]);
}
// B fragments for two adjacent n-tiles (8 rows each, rows n0.. and n0+8..) from a tile stored [n][k] (k contiguous)
__device__ __forceinline__ void load_b_nk(uint32_t sbase, int n0, int ks, uint32_t (&b)[4]) {
  const int lane = threadIdx.x & 31, mi = lane >> 3;
  ldsm4(tile_addr(sbase, n0 + (mi >> 1) * 8 + (lane & 7), ks * 2 + (mi & 1)), b[0], b[1], b[2], b[3]);   // {b0,b1} n-tile 0, {b2,b3} n-tile 1
}
// B fragments for two adjacent n-tiles (columns nc*8.. and nc*8+8..) from a tile stored [k][n] (n contiguous), k rows k0..k0+15
__device__ __forceinline__ void load_b_kn(uint32_t sbase, int k0, int nc, uint32_t (&b)[4]) {
  const int lane = threadIdx.x & 31, mi = lane >> 3;
  ldsm4t(tile_addr(sbase, k0 + (mi & 1) * 8 + (lane & 7), nc + (mi >> 1)), b[0], b[1], b[2], b[3]);
}
// store a warp's 16 x 64 fp32 accumulator tile (8 n-tiles) as bf16 into its own 16 rows of a swizzled tile, then to global
__device__ __forceinline__ void store_slab(uint32_t sbase, unsigned char* sgen, int row0, const float (&acc)[8][4], float scale0, float scale1,
                                           bf16* g, int ld, int grow0, int gcol0) {
  const int lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
  (void)sbase;
#pragma unroll
  for (int nt = 0; nt < 8; nt++) {
    const int r0 = row0 + gq, r1 = r0 + 8;
    *reinterpret_cast<uint32_t*>(sgen + r0 * 128 + ((nt ^ (r0 & 7)) << 4) + tq * 4) = pack2(acc[nt][0] * scale0, acc[nt][1] * scale0);
    *reinterpret_cast<uint32_t*>(sgen + r1 * 128 + ((nt ^ (r1 & 7)) << 4) + tq * 4) = pack2(acc[nt][2] * scale1, acc[nt][3] * scale1);
  }
  __syncwarp();
#pragma unroll
  for (int it = 0; it < 4; it++) {
    const int r = row0 + it * 4 + (lane >> 3), c = lane & 7;
    const uint4 v = *reinterpret_cast<const uint4*>(sgen + r * 128 + ((c ^ (r & 7)) << 4));
    *reinterpret_cast<uint4*>(g + (size_t)(grow0 + r - row0 + 0) * ld + gcol0 + c * 8) = v;
  }
}

// ---------------------------------------------------------------------------------------------- forward
// Task (b, h, qt): 128 query rows q0 = qt*128; writes o[N, D] (bf16) and lse[B, H, T].
__device__ __noinline__ void fwd_task(const bf16* qkv, bf16* o, float* lse, int b, int h, int qt, int T, int H, unsigned char* smem) {
  const int D = H * DH, ld = 3 * D;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gq = lane >> 2, tq = lane & 3;
  const uint32_t sQ = smem_u32(smem), sKV = sQ + QTILE * 128;     // stage s: K at sKV + s*16384, V at +8192
  const int q0 = qt * QTILE, nrow0 = b * T;
  const int nkt = (q0 + QTILE) / KTILE;
  load_tile(sQ, qkv, ld, nrow0 + q0, h * DH, QTILE);
  load_tile(sKV, qkv, ld, nrow0, D + h * DH, KTILE);
  load_tile(sKV + 8192, qkv, ld, nrow0, 2 * D + h * DH, KTILE);
  cp_async_commit();
  float oacc[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int wrow = q0 + warp * 16;              // first query row of this warp
  for (int kt = 0; kt < nkt; kt++) {
    const uint32_t sK = sKV + (kt & 1) * 16384, sV = sK + 8192;
    if (kt + 1 < nkt) {
      const uint32_t nK = sKV + ((kt + 1) & 1) * 16384;
      load_tile(nK, qkv, ld, nrow0 + (kt + 1) * KTILE, D + h * DH, KTILE);
      load_tile(nK + 8192, qkv, ld, nrow0 + (kt + 1) * KTILE, 2 * D + h * DH, KTILE);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int k0 = kt * KTILE;
    if (k0 <= wrow + 15) {                      // otherwise every key of the tile is in the future of every row of the warp
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; i++) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < 4; ks++) {
        uint32_t a[4]; load_a(sQ, warp * 16, ks, a);
#pragma unroll
        for (int np = 0; np < 4; np++) {
          uint32_t bb[4]; load_b_nk(sK, np * 16, ks, bb);
          mma16816(s[2 * np], a, bb[0], bb[1]);
          mma16816(s[2 * np + 1], a, bb[2], bb[3]);
        }
      }
      const bool need_mask = k0 + KTILE - 1 > wrow;
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; nt++) {
#pragma unroll
        for (int j = 0; j < 4; j++) {
          float v = s[nt][j] * SCALE_LOG2;
          if (need_mask) {
            const int kj = k0 + nt * 8 + tq * 2 + (j & 1), qi = wrow + gq + (j >> 1) * 8;
            if (kj > qi) v = -INFINITY;
          }
          s[nt][j] = v;
        }
        mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1])); mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float c0 = exp2f(m0 - mn0), c1 = exp2f(m1 - mn1);
      m0 = mn0; m1 = mn1;
      float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; nt++) {
        s[nt][0] = exp2f(s[nt][0] - mn0); s[nt][1] = exp2f(s[nt][1] - mn0);
        s[nt][2] = exp2f(s[nt][2] - mn1); s[nt][3] = exp2f(s[nt][3] - mn1);
        rs0 += s[nt][0] + s[nt][1]; rs1 += s[nt][2] + s[nt][3];
      }
      l0 = l0 * c0 + rs0; l1 = l1 * c1 + rs1;
#pragma unroll
      for (int i = 0; i < 8; i++) { oacc[i][0] *= c0; oacc[i][1] *= c0; oacc[i][2] *= c1; oacc[i][3] *= c1; }
#pragma unroll
      for (int kk = 0; kk < 4; kk++) {           // 16 keys per step
        uint32_t a[4];
        a[0] = pack2(s[2 * kk][0], s[2 * kk][1]); a[1] = pack2(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack2(s[2 * kk + 1][0], s[2 * kk + 1][1]); a[3] = pack2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < 4; dp++) {
          uint32_t bb[4]; load_b_kn(sV, kk * 16, dp * 2, bb);
          mma16816(oacc[2 * dp], a, bb[0], bb[1]);
          mma16816(oacc[2 * dp + 1], a, bb[2], bb[3]);
        }
      }
    }
    __syncthreads();
  }
  // row sums live spread over the 4 lanes of a quad
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = 1.f / l0, i1 = 1.f / l1;
  store_slab(sQ, smem, warp * 16, oacc, i0, i1, o, D, nrow0 + wrow, h * DH);
  if (tq == 0) {
    float* L = lse + ((size_t)b * H + h) * T;
    L[wrow + gq] = m0 * LN2 + logf(l0);
    L[wrow + gq + 8] = m1 * LN2 + logf(l1);
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------------- backward: prep
// Dr[b,h,t] = sum_d dO[n, h*64+d] * O[n, h*64+d]. Task (b, h, rt) covers 128 rows; two threads per row.
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

// ---------------------------------------------------------------------------------------------- backward: dK, dV
// Task (b, h, kt): 128 key rows k0 = kt*128 (16 per warp); walks query blocks of 64 rows from the diagonal to the end.
__device__ __noinline__ void bwd_dkdv_task(const bf16* qkv, const bf16* dO, const float* lse, const float* Dr, bf16* dqkv,
                                              int b, int h, int kt, int T, int H, unsigned char* smem) {
  const int D = H * DH, ld = 3 * D;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gq = lane >> 2, tq = lane & 3;
  const uint32_t sK = smem_u32(smem), sV = sK + QTILE * 128, sQd = sV + QTILE * 128;   // stage s: Q at sQd + s*16384, dO at +8192
  float* sStat = reinterpret_cast<float*>(smem + 2 * QTILE * 128 + 2 * 16384);          // stage s: lse at [s*128 .. +64), D at [s*128+64 ..)
  const int k0 = kt * QTILE, nrow0 = b * T;
  const int qb0 = k0 / KTILE, nqb = T / KTILE;
  const float* Lg = lse + ((size_t)b * H + h) * T;
  const float* Dg = Dr + ((size_t)b * H + h) * T;
  auto load_q = [&](int stage, int qb) {
    const uint32_t q = sQd + stage * 16384;
    load_tile(q, qkv, ld, nrow0 + qb * KTILE, h * DH, KTILE);
    load_tile(q + 8192, dO, D, nrow0 + qb * KTILE, h * DH, KTILE);
    if (tid < 32) {   // 64 lse + 64 D floats = 32 x 16 B
      const int which = tid >> 4, c = tid & 15;
      cp_async16(smem_u32(sStat + stage * 128 + which * 64 + c * 4), (which ? Dg : Lg) + qb * KTILE + c * 4);
    }
  };
  load_tile(sK, qkv, ld, nrow0 + k0, D + h * DH, QTILE);
  load_tile(sV, qkv, ld, nrow0 + k0, 2 * D + h * DH, QTILE);
  load_q(0, qb0);
  cp_async_commit();
  float dk[8][4], dv[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++) { dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f; dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f; }
  const int wkey = k0 + warp * 16;
  for (int qb = qb0; qb < nqb; qb++) {
    const int stage = (qb - qb0) & 1;
    const uint32_t sQ = sQd + stage * 16384, sdO = sQ + 8192;
    const float* sL = sStat + stage * 128; const float* sD = sL + 64;
    if (qb + 1 < nqb) { load_q(stage ^ 1, qb + 1); cp_async_commit(); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
#pragma unroll 1
    for (int qh = 0; qh < 2; qh++) {
      const int qbase = qb * KTILE + qh * 32;           // first query of this half
      if (qbase + 31 < wkey) continue;                  // all queries precede all keys of this warp
      float st[4][4], dpt[4][4];
#pragma unroll
      for (int i = 0; i < 4; i++) { st[i][0] = st[i][1] = st[i][2] = st[i][3] = 0.f; dpt[i][0] = dpt[i][1] = dpt[i][2] = dpt[i][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < 4; ks++) {
        uint32_t a[4], bb[4];
        load_a(sK, warp * 16, ks, a);
#pragma unroll
        for (int np = 0; np < 2; np++) {
          load_b_nk(sQ, qh * 32 + np * 16, ks, bb);
          mma16816(st[2 * np], a, bb[0], bb[1]); mma16816(st[2 * np + 1], a, bb[2], bb[3]);
        }
        load_a(sV, warp * 16, ks, a);
#pragma unroll
        for (int np = 0; np < 2; np++) {
          load_b_nk(sdO, qh * 32 + np * 16, ks, bb);
          mma16816(dpt[2 * np], a, bb[0], bb[1]); mma16816(dpt[2 * np + 1], a, bb[2], bb[3]);
        }
      }
      const bool need_mask = qbase < wkey + 16;
      uint32_t pa[2][4], da[2][4];                      // P^T and dS^T as bf16 A fragments (k = queries, 2 steps of 16)
#pragma unroll
      for (int nt = 0; nt < 4; nt++) {
        float p[4], ds[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const int ql = qh * 32 + nt * 8 + tq * 2 + (j & 1);          // query index inside the 64-block
          float pv = exp2f(st[nt][j] * SCALE_LOG2 - sL[ql] * LOG2E);
          if (need_mask) {
            const int kj = wkey + gq + (j >> 1) * 8, qi = qb * KTILE + ql;
            if (kj > qi) pv = 0.f;
          }
          p[j] = pv;
          ds[j] = pv * (dpt[nt][j] - sD[ql]);
        }
        pa[nt >> 1][(nt & 1) * 2] = pack2(p[0], p[1]); pa[nt >> 1][(nt & 1) * 2 + 1] = pack2(p[2], p[3]);
        da[nt >> 1][(nt & 1) * 2] = pack2(ds[0], ds[1]); da[nt >> 1][(nt & 1) * 2 + 1] = pack2(ds[2], ds[3]);
      }
#pragma unroll
      for (int kk = 0; kk < 2; kk++) {
#pragma unroll
        for (int dp = 0; dp < 4; dp++) {
          uint32_t bb[4];
          load_b_kn(sdO, qh * 32 + kk * 16, dp * 2, bb);
          mma16816(dv[2 * dp], pa[kk], bb[0], bb[1]); mma16816(dv[2 * dp + 1], pa[kk], bb[2], bb[3]);
          load_b_kn(sQ, qh * 32 + kk * 16, dp * 2, bb);
          mma16816(dk[2 * dp], da[kk], bb[0], bb[1]); mma16816(dk[2 * dp + 1], da[kk], bb[2], bb[3]);
        }
      }
    }
    __syncthreads();
  }
  store_slab(sK, smem, warp * 16, dk, SCALE, SCALE, dqkv, ld, nrow0 + wkey, D + h * DH);
  store_slab(sV, smem + QTILE * 128, warp * 16, dv, 1.f, 1.f, dqkv, ld, nrow0 + wkey, 2 * D + h * DH);
  __syncthreads();
}

// ---------------------------------------------------------------------------------------------- backward: dQ
// Task (b, h, qt): 128 query rows (16 per warp); walks key tiles of 64 rows from 0 to the diagonal.
__device__ __noinline__ void bwd_dq_task(const bf16* qkv, const bf16* dO, const float* lse, const float* Dr, bf16* dqkv,
                                            int b, int h, int qt, int T, int H, unsigned char* smem) {
  const int D = H * DH, ld = 3 * D;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gq = lane >> 2, tq = lane & 3;
  const uint32_t sQ = smem_u32(smem), sdO = sQ + QTILE * 128, sKV = sdO + QTILE * 128;
  const int q0 = qt * QTILE, nrow0 = b * T;
  const int nkt = (q0 + QTILE) / KTILE;
  load_tile(sQ, qkv, ld, nrow0 + q0, h * DH, QTILE);
  load_tile(sdO, dO, D, nrow0 + q0, h * DH, QTILE);
  load_tile(sKV, qkv, ld, nrow0, D + h * DH, KTILE);
  load_tile(sKV + 8192, qkv, ld, nrow0, 2 * D + h * DH, KTILE);
  cp_async_commit();
  const int wrow = q0 + warp * 16;
  const float* Lg = lse + ((size_t)b * H + h) * T;
  const float* Dg = Dr + ((size_t)b * H + h) * T;
  const float ls0 = Lg[wrow + gq] * LOG2E, ls1 = Lg[wrow + gq + 8] * LOG2E;
  const float dr0 = Dg[wrow + gq], dr1 = Dg[wrow + gq + 8];
  float dq[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++) { dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f; }
  for (int kt = 0; kt < nkt; kt++) {
    const uint32_t sK = sKV + (kt & 1) * 16384, sV = sK + 8192;
    if (kt + 1 < nkt) {
      const uint32_t nK = sKV + ((kt + 1) & 1) * 16384;
      load_tile(nK, qkv, ld, nrow0 + (kt + 1) * KTILE, D + h * DH, KTILE);
      load_tile(nK + 8192, qkv, ld, nrow0 + (kt + 1) * KTILE, 2 * D + h * DH, KTILE);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
#pragma unroll 1
    for (int kh = 0; kh < 2; kh++) {
      const int kbase = kt * KTILE + kh * 32;
      if (kbase > wrow + 15) continue;
      float s[4][4], dp[4][4];
#pragma unroll
      for (int i = 0; i < 4; i++) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < 4; ks++) {
        uint32_t a[4], bb[4];
        load_a(sQ, warp * 16, ks, a);
#pragma unroll
        for (int np = 0; np < 2; np++) {
          load_b_nk(sK, kh * 32 + np * 16, ks, bb);
          mma16816(s[2 * np], a, bb[0], bb[1]); mma16816(s[2 * np + 1], a, bb[2], bb[3]);
        }
        load_a(sdO, warp * 16, ks, a);
#pragma unroll
        for (int np = 0; np < 2; np++) {
          load_b_nk(sV, kh * 32 + np * 16, ks, bb);
          mma16816(dp[2 * np], a, bb[0], bb[1]); mma16816(dp[2 * np + 1], a, bb[2], bb[3]);
        }
      }
      const bool need_mask = kbase + 31 > wrow;
      uint32_t da[2][4];
#pragma unroll
      for (int nt = 0; nt < 4; nt++) {
        float ds[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          float pv = exp2f(s[nt][j] * SCALE_LOG2 - ((j >> 1) ? ls1 : ls0));
          if (need_mask) {
            const int kj = kbase + nt * 8 + tq * 2 + (j & 1), qi = wrow + gq + (j >> 1) * 8;
            if (kj > qi) pv = 0.f;
          }
          ds[j] = pv * (dp[nt][j] - ((j >> 1) ? dr1 : dr0));
        }
        da[nt >> 1][(nt & 1) * 2] = pack2(ds[0], ds[1]); da[nt >> 1][(nt & 1) * 2 + 1] = pack2(ds[2], ds[3]);
      }
#pragma unroll
      for (int kk = 0; kk < 2; kk++) {
#pragma unroll
        for (int dpi = 0; dpi < 4; dpi++) {
          uint32_t bb[4];
          load_b_kn(sK, kh * 32 + kk * 16, dpi * 2, bb);
          mma16816(dq[2 * dpi], da[kk], bb[0], bb[1]); mma16816(dq[2 * dpi + 1], da[kk], bb[2], bb[3]);
        }
      }
    }
    __syncthreads();
  }
  store_slab(sQ, smem, warp * 16, dq, SCALE, SCALE, dqkv, ld, nrow0 + wrow, h * DH);
  __syncthreads();
}

}  // namespace attn
}  // namespace ofa
