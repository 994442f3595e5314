// Host runtime behind the C ABI (include/ofa_b200.h): configuration, the flat parameter layout, device buffers, the
// builder of the training and serving phase graphs, TMA descriptor encoding, the one persistent launch and the result
// read-back. It is what main() of the reference program does (llm/b200/megakernel/ofa.cu:394-766), restructured as a
// library: nothing here exits the process or blocks without a bound.
#include "../../include/ofa_b200.h"
#include "megakernel.cuh"
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <string>
#include <vector>
#include <map>
#include <algorithm>

using namespace ofa;

namespace {

thread_local std::string g_create_error;
unsigned g_task_shuffle_seed = 0;   // test hook (ofa_debug_set_task_shuffle): != 0 -> the tickets of every phase uploaded from now on run their tasks in a permuted order

int gcd_int(int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; }
// multiplier in [2, n) coprime with n (0 = identity for phases too small to permute)
int shuffle_multiplier(unsigned seed, int phase, int n) {
  if (!seed || n < 3) return 0;
  int a = (int)((seed * 2654435761u + (unsigned)phase * 40503u) % (unsigned)n);
  for (int tries = 0; tries < n; tries++, a++) {
    if (a >= n) a = 2;
    if (a >= 2 && gcd_int(a, n) == 1) return a;
  }
  return 0;
}

struct HostPhase { std::string name; PhaseDesc d; std::vector<Dep> deps; std::vector<char> rb_grain;   // per dependency: 1 = wait per 128-token row block instead of for the whole producer phase
                   int rb_map = 0; };                                                                   // how this phase's tasks map to row blocks (RbKind | a << 8), 0 = they do not

struct DevJob {
  Job j{};
  PhaseDesc* ph = nullptr; SchedRec* rec = nullptr; int *prefix = nullptr, *ntasks = nullptr, *dep_off = nullptr, *dep_cnt = nullptr; Dep* deps = nullptr;
  int* done = nullptr; int* done_rb = nullptr; unsigned* ticket = nullptr;
  int nph = 0;
  std::vector<SchedRec> hrec;   // host copy of the scheduling records: they also travel inside the kernel parameter when they fit
  void free_all() {
    cudaFree(ph); cudaFree(rec); rec = nullptr; cudaFree(prefix); cudaFree(ntasks); cudaFree(dep_off); cudaFree(dep_cnt); cudaFree(deps); cudaFree(done); cudaFree(done_rb); cudaFree(ticket);
    *this = DevJob();
  }
};

struct Span { size_t off, n; };

struct Layout {   // flat parameter order: wte, wpe, [lm_head], per layer {g1, Wqkv, Wo, g2, Wup, Wdn}, gf
  size_t wte, wpe, head, gf, total;
  std::vector<size_t> g1, wqkv, wo, g2, wup, wdn;
  bool tied;
  std::map<std::string, Span> spans;
  void build(const ModelDims& m, bool tied_) {
    tied = tied_;
    size_t o = 0;
    const size_t D = m.D, V = m.V, T = m.T, FF = m.FF;
    auto add = [&](const std::string& nm, size_t n) { const size_t at = o; spans[nm] = Span{at, n}; o += n; return at; };
    wte = add("wte", V * D); wpe = add("wpe", T * D);
    head = tied ? wte : add("lm_head", V * D);
    if (tied) spans["lm_head"] = spans["wte"];
    for (int l = 0; l < m.L; l++) {
      const std::string p = "L" + std::to_string(l) + ".";
      g1.push_back(add(p + "g1", D)); wqkv.push_back(add(p + "Wqkv", D * 3 * D)); wo.push_back(add(p + "Wo", D * D));
      g2.push_back(add(p + "g2", D)); wup.push_back(add(p + "Wup", D * FF)); wdn.push_back(add(p + "Wdn", FF * D));
    }
    gf = add("gf", D);
    total = o;
  }
};

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                             const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn get_encode() {
  static EncodeFn enc = nullptr;
  if (!enc) {
    void* fn = nullptr; cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    enc = (EncodeFn)fn;
  }
  return enc;
}
// 2-D tensor map: `inner` contiguous elements, `outer` rows of `ld` elements, box {box_inner, box_outer}. GEMM operands are
// bf16 with SWIZZLE_128B; the serving job's weight prefetch uses plain (unswizzled) views in the activation type.
bool encode_map(CUtensorMap* m, const void* base, uint64_t inner, uint64_t outer, uint64_t ld, uint32_t box_inner, uint32_t box_outer,
                bool is_f32 = false, bool swizzle = true) {
  EncodeFn enc = get_encode();
  if (!enc) return false;
  cuuint64_t dims[2] = {inner, outer}, strides[1] = {ld * (is_f32 ? 4u : 2u)};
  cuuint32_t box[2] = {box_inner, box_outer}, es[2] = {1, 1};
  return enc(m, is_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
             swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Arena {   // device allocations owned by one context / one ofa_run_phases call
  std::vector<void*> ptrs;
  bool ok = true;
  bool dry = false;            // planning mode (no device): hands out distinct, aligned, never-dereferenced addresses
  uintptr_t bump = 0x100000000ull;
  template <class T> T* alloc(size_t n, bool zero = true) {
    void* p = nullptr;
    if (n == 0) n = 1;
    if (dry) { p = reinterpret_cast<void*>(bump); bump += (n * sizeof(T) + 1023) / 1024 * 1024; return reinterpret_cast<T*>(p); }
    if (cudaMalloc(&p, n * sizeof(T)) != cudaSuccess) { ok = false; return nullptr; }
    if (zero) cudaMemset(p, 0, n * sizeof(T));
    ptrs.push_back(p);
    return reinterpret_cast<T*>(p);
  }
  void h2d(void* dst, const void* src, size_t bytes) { if (!dry) cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice); }
  void free_all() { for (void* p : ptrs) cudaFree(p); ptrs.clear(); }
};

// TMA descriptors of one layer's attention operands (qkv [N, 3D] and, for the backward tasks, dO [N, D]) in device memory
const void* make_attn_maps(Arena& ar, const void* qkv, const void* dO, int N, int D, std::string& err) {
  attn_tc::Maps* dm = ar.alloc<attn_tc::Maps>(1, false);
  if (ar.dry || !dm) return dm;
  attn_tc::Maps hm; memset(&hm, 0, sizeof hm);
  bool ok = encode_map(&hm.qkv128, qkv, 3 * D, N, 3 * D, 64, 128) && encode_map(&hm.qkv64, qkv, 3 * D, N, 3 * D, 64, 64);
  if (dO) ok = ok && encode_map(&hm.dO128, dO, D, N, D, 64, 128) && encode_map(&hm.dO64, dO, D, N, D, 64, 64);
  if (!ok) { err = "cuTensorMapEncodeTiled failed (attention)"; return nullptr; }
  ar.h2d(dm, &hm, sizeof hm);
  return dm;
}

// Validates a GEMM description for the tensor-core path and fills task counts + TMA descriptors (device memory).
bool prepare_gemm_bf16(PhaseDesc& d, Arena& ar, int nsub_cfg, int nblocks, std::string& err) {
  GemmArgs& g = d.g;
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (g.M <= 0 || g.N <= 0 || g.K <= 0 || g.M % 128 || g.N % 128 || g.K % 64 || g.lda % 8 || g.ldb % 8 || g.ldc % 8 ||
      !al16(g.A) || !al16(g.B) || !al16(g.C) || (g.aux && (!al16(g.aux) || g.ldaux % 8))) {
    err = "GEMM needs M,N % 128 == 0, K % 64 == 0, leading dimensions % 8 == 0 and 16-byte aligned pointers";
    return false;
  }
  if ((d.epi == GE_RES || d.epi == GE_GELU || d.epi == GE_DGELU || d.epi == GE_DR) && !g.aux) { err = "GEMM epilogue needs aux"; return false; }
  if (d.epi == GE_LSE && (d.layout != GL_NT || !g.dr)) { err = "softmax-partial epilogue: NT layout with an output for the partials"; return false; }
  // nsub_cfg: n = strips of n tiles (0 = automatic); 2000 + n = the same with 256-wide tiles where N allows. 256-wide tiles are
  // opt-in: with two 48 KB stages per block they measured slower than three 32 KB stages of the 128-wide tile on every model
  // shape except lm_head dW (960 vs 702 TFLOP/s), i.e. the main loop is bound by bytes in flight, not by operand traffic alone.
  const bool nfast = nsub_cfg >= 4000;             // 4000 + n: 256-wide tiles and tasks ordered along N first (see gemm_tc_task)
  if (nfast) nsub_cfg -= 2000;
  d.i0 = nfast ? 1 : 0;
  const bool want256 = nsub_cfg >= 2000;
  if (want256) nsub_cfg -= 2000;
  g.bn = (want256 && g.N % 256 == 0 && d.epi != GE_DR && d.epi != GE_LSE) ? 256 : 128;
  const int tm = g.M / 128, tn = g.N / g.bn;
  int nsub = nsub_cfg;
  if (nsub <= 0) {
    // strip length: fewest waves of the resident blocks, then the most tasks (a strip pays pipeline fill, drain and the claim once)
    const int kt = g.K / 64;
    double best = 1e30; nsub = 1;
    for (int c = 1; c <= std::min(tn, 8); c++) {
      const long tasks = (long)tm * ((tn + c - 1) / c);
      const long waves = (tasks + nblocks - 1) / nblocks;
      const double per_k = g.bn == 256 ? 0.9 : 0.66;           // us per 64-deep K step of one block with the GPU busy (measured)
      const double cost = waves * (5.0 + c * kt * per_k);
      if (cost < best - 1e-9) { best = cost; nsub = c; }
    }
  }
  nsub = std::max(1, std::min(nsub, tn));
  g.nsub = nsub;
  d.tiles_m = tm;
  d.ntasks = tm * ((tn + nsub - 1) / nsub);
  if (ar.dry) { g.tmA = ar.alloc<CUtensorMap>(2, false); g.tmB = reinterpret_cast<const CUtensorMap*>(g.tmA) + 1; return true; }
  CUtensorMap hm[2];
  const bool a_kmajor = d.layout != GL_TN, b_kmajor = d.layout == GL_NT;
  bool ok = a_kmajor ? encode_map(&hm[0], g.A, g.K, g.M, g.lda, 64, 128) : encode_map(&hm[0], g.A, g.M, g.K, g.lda, 64, 64);
  ok = ok && (b_kmajor ? encode_map(&hm[1], g.B, g.K, g.N, g.ldb, 64, 128) : encode_map(&hm[1], g.B, g.N, g.K, g.ldb, 64, 64));
  if (!ok) { err = "cuTensorMapEncodeTiled failed"; return false; }
  CUtensorMap* dm = ar.alloc<CUtensorMap>(2, false);
  if (!dm) { err = "cudaMalloc failed"; return false; }
  cudaMemcpy(dm, hm, sizeof hm, cudaMemcpyHostToDevice);
  g.tmA = dm; g.tmB = dm + 1;
  return true;
}
void prepare_gemm_f32(PhaseDesc& d) {
  d.tiles_m = (d.g.M + f32::GT - 1) / f32::GT;
  d.ntasks = d.tiles_m * ((d.g.N + f32::GT - 1) / f32::GT);
  d.g.nsub = 1;
}

// nrb = number of 128-token row blocks (0: no phase counts completions per row block, every dependency is phase-level)
bool upload_job(const std::vector<HostPhase>& ph, int last_phase, int nsteps, DevJob& dj, std::string& err, int nrb = 0) {
  const int nph = (int)ph.size();
  std::vector<PhaseDesc> pd(nph); std::vector<int> prefix(nph + 1, 0), nt(nph), doff(nph), dcnt(nph); std::vector<Dep> deps;
  for (int i = 0; i < nph; i++) {
    pd[i] = ph[i].d; nt[i] = ph[i].d.ntasks; prefix[i + 1] = prefix[i] + nt[i];
    doff[i] = (int)deps.size(); dcnt[i] = (int)ph[i].deps.size();
    for (const Dep& e : ph[i].deps) {
      if (e.phase < 0 || e.phase >= nph || (e.delta == 0 && e.phase >= i) || e.delta > 0 || e.delta < -1) { err = "bad dependency in phase " + ph[i].name; return false; }
      deps.push_back(e);
    }
    if (nt[i] <= 0) { err = "phase without tasks: " + ph[i].name; return false; }
  }
  if ((double)prefix[nph] * (double)nsteps >= 4.0e9) { err = "ticket counter would overflow"; return false; }
  if (nph >= 65536) { err = "too many phases"; return false; }
  // which phases count their completions per row block: those that say how their tasks map to row blocks, have a whole number of
  // tasks per row block, and are waited for at that grain by somebody
  std::vector<int> rb_off(nph, -1); int rb_total = 0;
  if (nrb > 0 && !getenv("OFA_B200_PHASE_DEPS"))           // A/B switch for measurements: phase-level dependencies only
    for (int i = 0; i < nph; i++)
      for (size_t k = 0; k < ph[i].deps.size() && ph[i].deps.size() <= 4; k++) {
        const int p = ph[i].deps[k].phase;
        if (k < ph[i].rb_grain.size() && ph[i].rb_grain[k] && ph[i].rb_map && ph[p].rb_map && nt[p] % nrb == 0 && rb_off[p] < 0) { rb_off[p] = rb_total; rb_total += nrb; }
      }
  std::vector<SchedRec> rec(nph);
  for (int i = 0; i < nph; i++) {
    SchedRec& r = rec[i]; memset(&r, 0, sizeof(r));
    r.lo = prefix[i]; r.hi = prefix[i + 1];
    const int n = (int)ph[i].deps.size();
    r.ndeps = n <= 4 ? n : -1;
    r.perm_mul = shuffle_multiplier(g_task_shuffle_seed, i, nt[i]);
    r.rb_off = rb_off[i]; r.rb_map = ph[i].rb_map;
    for (int k = 0; k < n && n <= 4; k++) {
      const Dep& e = ph[i].deps[k];
      const bool rb = k < (int)ph[i].rb_grain.size() && ph[i].rb_grain[k] && ph[i].rb_map && rb_off[e.phase] >= 0;
      r.dep[2 * k] = e.phase | (e.delta == -1 ? DEP_PREV : 0) | (rb ? DEP_RB : 0);
      r.dep[2 * k + 1] = rb ? nt[e.phase] / nrb : nt[e.phase];
    }
  }
  if (deps.empty()) deps.push_back(Dep{0, 0});
  dj.free_all();
  bool ok = cudaMalloc(&dj.ph, sizeof(PhaseDesc) * nph) == cudaSuccess && cudaMalloc(&dj.prefix, 4 * (nph + 1)) == cudaSuccess &&
            cudaMalloc(&dj.ntasks, 4 * nph) == cudaSuccess && cudaMalloc(&dj.dep_off, 4 * nph) == cudaSuccess &&
            cudaMalloc(&dj.dep_cnt, 4 * nph) == cudaSuccess && cudaMalloc(&dj.deps, sizeof(Dep) * deps.size()) == cudaSuccess &&
            cudaMalloc(&dj.done, 4 * nph) == cudaSuccess && cudaMalloc(&dj.ticket, 4) == cudaSuccess &&
            cudaMalloc(&dj.rec, sizeof(SchedRec) * nph) == cudaSuccess && cudaMalloc(&dj.done_rb, 4 * (size_t)std::max(1, rb_total)) == cudaSuccess;
  if (!ok) { err = "cudaMalloc failed (job tables)"; return false; }
  cudaMemcpy(dj.ph, pd.data(), sizeof(PhaseDesc) * nph, cudaMemcpyHostToDevice);
  cudaMemcpy(dj.rec, rec.data(), sizeof(SchedRec) * nph, cudaMemcpyHostToDevice);
  cudaMemcpy(dj.prefix, prefix.data(), 4 * (nph + 1), cudaMemcpyHostToDevice);
  cudaMemcpy(dj.ntasks, nt.data(), 4 * nph, cudaMemcpyHostToDevice);
  cudaMemcpy(dj.dep_off, doff.data(), 4 * nph, cudaMemcpyHostToDevice);
  cudaMemcpy(dj.dep_cnt, dcnt.data(), 4 * nph, cudaMemcpyHostToDevice);
  cudaMemcpy(dj.deps, deps.data(), sizeof(Dep) * deps.size(), cudaMemcpyHostToDevice);
  cudaMemset(dj.done, 0, 4 * nph); cudaMemset(dj.ticket, 0, 4); cudaMemset(dj.done_rb, 0, 4 * (size_t)std::max(1, rb_total));
  dj.nph = nph; dj.hrec = rec;
  dj.j.nph = nph; dj.j.tasks_per_step = prefix[nph]; dj.j.nsteps = nsteps; dj.j.last_phase = last_phase;
  dj.j.ph = dj.ph; dj.j.prefix = dj.prefix; dj.j.ntasks = dj.ntasks; dj.j.dep_off = dj.dep_off; dj.j.dep_cnt = dj.dep_cnt; dj.j.deps = dj.deps; dj.j.rec = dj.rec;
  dj.j.done = dj.done; dj.j.done_rb = dj.done_rb; dj.j.ticket = dj.ticket;
  return true;
}

// copies a job's scheduling records into the kernel parameter when they fit
void fill_param_records(Ctx& C, const DevJob* train, const DevJob* dec) {
  C.train_rec_n = 0; C.dec_rec_n = 0;
  C.sched_flags = getenv("OFA_B200_LATE_TICKETS") ? 4 : 0;     // A/B switch for measurements: tickets only at the end of a task
  if (getenv("OFA_B200_GLOBAL_RECS")) return;      // A/B switch for measurements: keep using the records in global memory
  if (train && train->nph > 0 && train->nph <= PARAM_TRAIN_PH) { memcpy(C.train_rec, train->hrec.data(), sizeof(SchedRec) * train->nph); C.train_rec_n = train->nph; }
  if (dec && dec->nph > 0 && dec->nph <= PARAM_DEC_PH) { memcpy(C.dec_rec, dec->hrec.data(), sizeof(SchedRec) * dec->nph); C.dec_rec_n = dec->nph; }
}

template <class T, int D, int DH> cudaError_t launch_kernel(const Ctx& C, int nblocks, int smem, cudaStream_t s) {
  cudaError_t e = cudaFuncSetAttribute(ofa_kernel<T, D, DH>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  // ask for the largest shared-memory carve-out on every SM: with a smaller split an SM holds one 113 KB block instead of two,
  // and a persistent block never leaves to let the split be changed (measured: 24 SMs ran with a single block)
  cudaFuncSetAttribute(ofa_kernel<T, D, DH>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  ofa_kernel<T, D, DH><<<nblocks, NTHR, smem, s>>>(C);
  return cudaGetLastError();
}

// Tasks whose shared-memory need grows with the batch or the context must fit the block's task area: on the bf16 path that is
// the fixed GEMM pipeline + staging region below the control area (an oversize task would overwrite the block's barriers and
// scheduler words, or store beyond the shared window); on the fp32 path the window is sized from them and must stay within
// the device's per-block opt-in limit. Returns an empty string when everything fits.
std::string smem_fit_error(bool bf, int Tctx, int N, bool emb_wte, bool decode, int smem) {
  if (bf) {
    const size_t room = gemm_tc::BAR_OFFSET;
    if (emb_wte && ew::embed_bwd_wte_smem_bytes(N) > room)
      return "batch * ctx_len = " + std::to_string(N) + " tokens: the embedding-backward task needs " + std::to_string(ew::embed_bwd_wte_smem_bytes(N)) + " B of shared memory, the block has " + std::to_string(room);
    if (decode && dec::smem_bytes<bf16, 768, 64>(Tctx) > room)
      return "ctx_len " + std::to_string(Tctx) + ": the serving tasks need " + std::to_string(dec::smem_bytes<bf16, 768, 64>(Tctx)) + " B of shared memory, the block has " + std::to_string(room);
    return "";
  }
  if (smem > 227 * 1024) return "the fp32 path would need " + std::to_string(smem) + " B of shared memory per block (limit 232,448)";
  return "";
}

int smem_for(bool bf, int Tctx, int N) {
  if (bf) return gemm_tc::SMEM_BYTES;
  size_t m = f32::GEMM_SMEM;
  m = std::max(m, f32::attn_bwd_smem(Tctx, 16));
  m = std::max(m, ew::embed_bwd_wte_smem_bytes(N));
  m = std::max(m, ew::ln_bwd_smem_bytes<64>());
  m = std::max(m, dec::smem_bytes<float, 64, 16>(Tctx));
  m = std::max(m, (size_t)64 + 4096);
  return (int)((m + 1023) / 1024 * 1024) + CTRL_BYTES;   // + control area
}

}  // namespace

// ================================================================================================ context
struct ofa_dp_state;
extern "C" void ofa_dp_shutdown(ofa_ctx* c);
struct ofa_ctx {
  ofa_dp_state* dp = nullptr;        // communication side of data parallelism (dp_nccl.inc), created by ofa_dp_init
  ofa_config cfg{};
  ModelDims md{};
  bool bf = true;
  Layout lay;
  int device = 0, num_sms = 0, nblocks = 0, smem = 0;
  Arena ar;
  float *W32 = nullptr, *G32 = nullptr, *M32 = nullptr, *V32 = nullptr; void* Wact = nullptr; bf16* Gbf = nullptr;
  uint32_t* d_tokens = nullptr; size_t ntok = 0; uint32_t* d_starts = nullptr; int nstarts = 0;
  std::map<std::string, std::pair<void*, size_t>> bufs;
  std::vector<HostPhase> train_ph, dec_ph; int train_last = 0, dec_last = 0;
  DevJob train_job, dec_job;
  Ctx C{};
  DevStatus* d_status = nullptr;
  int* d_finished = nullptr; unsigned long long* d_t_end = nullptr;
  unsigned long long *d_phase_busy = nullptr, *d_phase_first = nullptr, *d_phase_last = nullptr, *d_step_done = nullptr, *d_blk_busy = nullptr;
  float* d_loss_hist = nullptr; int loss_cap = 0;
  unsigned long long* d_dec_phase_busy = nullptr; int* d_blk_info = nullptr;
  int* d_smid_rank = nullptr;
  Live* h_live = nullptr; Live* d_live = nullptr;
  int* h_out = nullptr; int* d_out = nullptr; int out_cap = 0;
  int* d_forced = nullptr; int* d_scal = nullptr;
  int* d_ext_ready = nullptr; int* d_ext_done = nullptr;   // device flags [32] each: gradients of bucket b ready / all-reduce of bucket b done
  std::vector<Span> buckets;
  cudaStream_t stream = nullptr, abort_stream = nullptr; cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  bool dry = false;
  int step_done_cap = 0; size_t starts_cap = 0, tokens_cap = 0;
  bool abort_requested = false;      // ofa_abort was called for the launch in flight (also honoured if the device word was cleared by a launch that had not started yet)
  bool in_flight = false; int steps_total = 0, last_nsteps = 0; float last_ms = 0.f; int dec_steps_total = 0;
  std::string err;
};

namespace {

int fail(ofa_ctx* c, int code, const std::string& msg) { if (c) c->err = msg; else g_create_error = msg; return code; }

template <class T> T* abuf(ofa_ctx* c, const std::string& name, size_t n) {
  T* p = c->ar.alloc<T>(n);
  c->bufs[name] = std::make_pair((void*)p, n * sizeof(T));
  return p;
}

// ---------------------------------------------------------------------------------------------- training graph
// Phase order and dependencies follow the reference graph (ofa.cu:548-645) with an untied LM head as an option: the
// head has its own AdamW phase, `logits` of the next step waits for it, and `lnf` of the next step waits for `head dW`
// (which still reads the lnf buffer). Every gradient tensor is overwritten by its single producer, so AdamW does not
// zero anything. With ext_sync the parameters are cut into contiguous gradient buckets; a 1-task "grads ready b" phase
// raises a flag when bucket b is complete and a 1-task "allreduce done b" phase holds that bucket's AdamW until the
// communication side has raised the matching flag.
struct Bucket { size_t off, n; std::vector<std::string> producers; std::vector<std::string> adam_phases; int last_layer; };

template <class T>
bool build_train_graph(ofa_ctx* c) {
  const ModelDims& m = c->md; const ofa_config& cfg = c->cfg; const Layout& lay = c->lay;
  const bool bf = c->bf;
  const size_t N = m.N, D = m.D, FF = m.FF, V = m.V;
  const int L = m.L;
  T* Wact = reinterpret_cast<T*>(c->Wact);
  std::vector<HostPhase>& P = c->train_ph;
  P.clear();
  std::map<std::string, int> id;
  std::vector<std::vector<std::string>> prevdeps;   // cross-step dependencies by name (targets may be defined later)
  std::string err;
  bool ok = true;
  // how a phase's tasks map to 128-token row blocks (tensor-core path only: its row counts are multiples of 128)
  const bool rb_ok = bf && m.N % 128 == 0 && m.T % 128 == 0;
  auto rbmap = [&](const PhaseDesc& d) -> int {
    if (!rb_ok) return 0;
    switch (d.kind) {
      case TK_GEMM: return (d.layout != GL_TN && d.g.M == (int)N && d.tiles_m == (int)N / 128) ? (RB_MOD | d.tiles_m << 8) : 0;
      case TK_LN_FWD: case TK_LN_BWD: case TK_EMBED: return RB_DIV | (128 / ew::ROWS_PER_TASK) << 8;
      case TK_CE: return RB_DIV | (128 / ew::CE_ROWS) << 8;
      case TK_ATT_FWD: return RB_ATT_FWD;
      case TK_ATT_BWD: return RB_ATT_BWD;
      default: return 0;
    }
  };
  // rbdeps: those of deps0 that are waited for per row block (the consumer task reads only the rows of its own row blocks)
  auto addp = [&](const std::string& name, const PhaseDesc& d, std::vector<std::string> deps0, std::vector<std::string> deps_prev, std::vector<std::string> rbdeps = {}) {
    HostPhase hp; hp.name = name; hp.d = d; hp.rb_map = rbmap(d);
    for (const std::string& e : deps0) {
      if (e.empty()) continue;
      auto it = id.find(e);
      if (it == id.end()) { ok = false; err = "unknown dependency " + e + " of " + name; continue; }
      bool dup = false; for (const Dep& x : hp.deps) dup = dup || x.phase == it->second;
      if (!dup) { hp.deps.push_back(Dep{it->second, 0}); hp.rb_grain.push_back(std::find(rbdeps.begin(), rbdeps.end(), e) != rbdeps.end() ? 1 : 0); }
    }
    id[name] = (int)P.size();
    P.push_back(hp);
    std::vector<std::string> pv; for (auto& e : deps_prev) if (!e.empty()) pv.push_back(e);
    prevdeps.push_back(pv);
  };
  auto mk = [&](int kind, int ntasks) { PhaseDesc d; memset(&d, 0, sizeof d); d.kind = kind; d.ntasks = ntasks; return d; };
  // wide = 1: 128 x 256 tiles where the width allows (a long K and more tiles than blocks: only the LM head's weight gradient)
  auto mkgemm = [&](int layout, int epi, const void* A, int lda, const void* B, int ldb, void* Cc, int ldc, void* aux, int ldaux,
                    int M, int Nn, int K, int accumulate, int wide = 0) {
    PhaseDesc d = mk(TK_GEMM, 0); d.layout = layout; d.epi = epi;
    d.g.A = A; d.g.B = B; d.g.C = Cc; d.g.aux = aux; d.g.M = M; d.g.N = Nn; d.g.K = K; d.g.lda = lda; d.g.ldb = ldb; d.g.ldc = ldc; d.g.ldaux = ldaux;
    d.g.accumulate = accumulate;
    // wide: 128 x 256 tiles, one tile per task, tasks ordered along N first (the three readers of a 128-row slice of the large
    // operand run side by side and share it through L2); OFA_B200_HEAD_DW_128 / _STRIPS keep the other two forms for A/B runs
    const int nsub_cfg = (wide && cfg.gemm_nsub == 0 && !getenv("OFA_B200_HEAD_DW_128")) ? (getenv("OFA_B200_HEAD_DW_STRIPS") ? 2000 : 4001) : cfg.gemm_nsub;
    if (bf) { std::string e; if (!prepare_gemm_bf16(d, c->ar, nsub_cfg, c->C.train_sms > 0 ? 2 * c->C.train_sms : c->nblocks, e)) { ok = false; err = e; } }   // waves are counted over the blocks that train
    else prepare_gemm_f32(d);
    return d;
  };
  const bool train = cfg.mode == OFA_MODE_TRAIN, fwd_only = cfg.mode == OFA_MODE_FORWARD;
  const bool gbf = cfg.grad_bf16 != 0;
  auto G = [&](size_t off) -> void* { return gbf ? (void*)(c->Gbf + off) : (void*)(c->G32 + off); };
  const int wepi = gbf ? GE_STORE : GE_F32;
  const int rows16 = (int)((N + 15) / 16);

  // ---- buffers (per layer, no aliasing: a layer's backward reads what its forward wrote)
  std::vector<T*> xs(L + 1), ln1(L), qkv(L), att(L), hb(L), ln2(L), upre(L), uact(L);
  std::vector<float*> mean1(L), rstd1(L), mean2(L), rstd2(L), lse(L), Dr(L), dgp1(L), dgp2(L);
  std::vector<T*> dxs(L + 1), dpre(L), dln2(L), dh(L), dob(L), dqkv(L), dln1(L);
  for (int l = 0; l <= L; l++) xs[l] = abuf<T>(c, "x" + std::to_string(l), N * D);
  for (int l = 0; l < L; l++) {
    const std::string s = std::to_string(l);
    ln1[l] = abuf<T>(c, "ln1_" + s, N * D); qkv[l] = abuf<T>(c, "qkv" + s, N * 3 * D); att[l] = abuf<T>(c, "att" + s, N * D);
    hb[l] = abuf<T>(c, "h" + s, N * D); ln2[l] = abuf<T>(c, "ln2_" + s, N * D); upre[l] = abuf<T>(c, "upre" + s, N * FF); uact[l] = abuf<T>(c, "uact" + s, N * FF);
    mean1[l] = abuf<float>(c, "mean1_" + s, N); rstd1[l] = abuf<float>(c, "rstd1_" + s, N); mean2[l] = abuf<float>(c, "mean2_" + s, N); rstd2[l] = abuf<float>(c, "rstd2_" + s, N);
    lse[l] = abuf<float>(c, "lse" + s, N * m.H);
  }
  T* lnf = abuf<T>(c, "lnf", N * D); float* meanf = abuf<float>(c, "meanf", N); float* rstdf = abuf<float>(c, "rstdf", N);
  T* logits = abuf<T>(c, "logits", N * V); float* lossv = abuf<float>(c, "lossv", N); float* meanloss = abuf<float>(c, "meanloss", 4);
  T* dxf = nullptr; float* dgpf = nullptr;
  if (!fwd_only) {
    for (int l = 0; l <= L; l++) dxs[l] = abuf<T>(c, "dx" + std::to_string(l), N * D);
    for (int l = 0; l < L; l++) {
      const std::string s = std::to_string(l);
      dpre[l] = abuf<T>(c, "dpre" + s, N * FF); dln2[l] = abuf<T>(c, "dln2_" + s, N * D); dh[l] = abuf<T>(c, "dh" + s, N * D); dob[l] = abuf<T>(c, "datt" + s, N * D);
      dqkv[l] = abuf<T>(c, "dqkv" + s, N * 3 * D); dln1[l] = abuf<T>(c, "dln1_" + s, N * D);
      Dr[l] = abuf<float>(c, "Dr" + s, N * m.H); dgp1[l] = abuf<float>(c, "dgp1_" + s, (size_t)rows16 * D); dgp2[l] = abuf<float>(c, "dgp2_" + s, (size_t)rows16 * D);
    }
    dxf = abuf<T>(c, "dxf", N * D); dgpf = abuf<float>(c, "dgpf", (size_t)rows16 * D);
  }
  c->C.tok_in = c->ar.alloc<int>(N); c->C.tok_tgt = c->ar.alloc<int>(N);
  if (!c->ar.ok) { c->err = "out of device memory (activations)"; return false; }

  const std::string step_end = "step barrier";
  const std::string opt_wte = train ? "adamw wte" : "", opt_wpe = train ? "adamw wpe" : "";
  const std::string opt_head = train ? (lay.tied ? "adamw wte" : "adamw head") : "";
  auto opt_layer = [&](int l) { return train ? "adamw L" + std::to_string(l) : std::string(); };

  // ---- forward
  { PhaseDesc d = mk(TK_DATA, m.B); addp("data", d, {}, {train ? std::string("embed bwd wte") : step_end}); }
  { PhaseDesc d = mk(TK_EMBED, rows16); d.p[0] = xs[0]; d.p[1] = Wact + lay.wte; d.p[2] = Wact + lay.wpe; d.p[3] = c->C.tok_in;
    addp("embed", d, {"data"}, {opt_wte, opt_wpe}); }
  std::string prev = "embed";
  const int attn_fwd_tasks = bf ? m.B * m.H * (m.T / attn::QTILE) : m.B * m.H;
  for (int l = 0; l < L; l++) {
    const std::string s = "L" + std::to_string(l) + " ";
    { PhaseDesc d = mk(TK_LN_FWD, rows16); d.p[0] = ln1[l]; d.p[1] = mean1[l]; d.p[2] = rstd1[l]; d.p[3] = xs[l]; d.p[4] = Wact + lay.g1[l];
      addp(s + "ln1", d, {prev}, {opt_layer(l)}, {prev}); }
    addp(s + "qkv", mkgemm(GL_NN, GE_STORE, ln1[l], D, Wact + lay.wqkv[l], 3 * D, qkv[l], 3 * D, nullptr, 0, N, 3 * D, D, 0), {s + "ln1"}, {}, {s + "ln1"});
    { PhaseDesc d = mk(TK_ATT_FWD, attn_fwd_tasks); d.p[0] = qkv[l]; d.p[1] = att[l]; d.p[2] = lse[l];
      if (bf) { std::string e; d.p[6] = const_cast<void*>(make_attn_maps(c->ar, qkv[l], nullptr, N, D, e)); if (!d.p[6]) { ok = false; err = e; } }
      addp(s + "attn", d, {s + "qkv"}, {}, {s + "qkv"}); }
    addp(s + "wo+res", mkgemm(GL_NN, GE_RES, att[l], D, Wact + lay.wo[l], D, hb[l], D, xs[l], D, N, D, D, 0), {s + "attn"}, {}, {s + "attn"});
    { PhaseDesc d = mk(TK_LN_FWD, rows16); d.p[0] = ln2[l]; d.p[1] = mean2[l]; d.p[2] = rstd2[l]; d.p[3] = hb[l]; d.p[4] = Wact + lay.g2[l];
      addp(s + "ln2", d, {s + "wo+res"}, {}, {s + "wo+res"}); }
    addp(s + "up+gelu", mkgemm(GL_NN, GE_GELU, ln2[l], D, Wact + lay.wup[l], FF, uact[l], FF, upre[l], FF, N, FF, D, 0), {s + "ln2"}, {}, {s + "ln2"});
    addp(s + "down+res", mkgemm(GL_NN, GE_RES, uact[l], FF, Wact + lay.wdn[l], D, xs[l + 1], D, hb[l], D, N, D, FF, 0), {s + "up+gelu"}, {}, {s + "up+gelu"});
    prev = s + "down+res";
  }
  { PhaseDesc d = mk(TK_LN_FWD, rows16); d.p[0] = lnf; d.p[1] = meanf; d.p[2] = rstdf; d.p[3] = xs[L]; d.p[4] = Wact + lay.gf;
    addp("lnf", d, {prev}, {fwd_only ? "" : "head dW"}, {prev}); }
  // Head fusion: with a backward pass behind it the LM-head GEMM also leaves, per row and 128-column tile, the maximum and the sum
  // of exponentials of the values it stored; cross-entropy then reads the logits once instead of twice (the reference reads them
  // in two passes, llm/elementwise/ew_loss.cuh:19-75).
  float2* lse_part = nullptr;
  const bool fuse_head = bf && !fwd_only && V % 128 == 0 && !getenv("OFA_B200_CE_TWO_PASS");     // the switch keeps the two-pass task for A/B measurements
  if (fuse_head) lse_part = reinterpret_cast<float2*>(abuf<float>(c, "lse_part", N * (V / 128) * 2));
  {
    PhaseDesc d = mk(TK_GEMM, 0); d.layout = GL_NT; d.epi = fuse_head ? GE_LSE : GE_STORE;
    d.g.A = lnf; d.g.B = Wact + lay.head; d.g.C = logits; d.g.aux = nullptr; d.g.M = (int)N; d.g.N = (int)V; d.g.K = (int)D; d.g.lda = (int)D; d.g.ldb = (int)D; d.g.ldc = (int)V;
    d.g.dr = reinterpret_cast<float*>(lse_part);
    if (bf) { std::string e; if (!prepare_gemm_bf16(d, c->ar, cfg.gemm_nsub, c->C.train_sms > 0 ? 2 * c->C.train_sms : c->nblocks, e)) { ok = false; err = e; } }
    else prepare_gemm_f32(d);
    addp("logits", d, {"lnf"}, {opt_head}, {"lnf"});
  }
  std::vector<std::string> end_deps;
  if (fwd_only) {
    end_deps = {"logits"};
  } else {
    { PhaseDesc d = mk(TK_CE, (int)((N + ew::CE_ROWS - 1) / ew::CE_ROWS)); d.p[0] = logits; d.p[1] = c->C.tok_tgt; d.p[2] = lossv; d.p[3] = lse_part; d.i2 = (int)(V / 128);
      const size_t usable = (size_t)((bf ? gemm_tc::BAR_OFFSET : c->smem - CTRL_BYTES) - 64);
      d.i0 = (int)(std::min(usable, V * sizeof(T)) / 16 * 16);
      addp("cross-entropy", d, {"logits", "data"}, {}, {"logits"}); }
    { PhaseDesc d = mk(TK_CE_MEAN, 1); d.p[0] = meanloss; d.p[1] = lossv; addp("loss mean", d, {"cross-entropy"}, {}); }

    // ---- gradient buckets (only used with ext_sync): head | layer groups from the top | wte+wpe
    std::vector<Bucket> buckets;
    std::vector<int> bucket_of_layer(L, -1);
    const bool ext = train && cfg.ext_sync != 0;
    if (ext) {
      const size_t esz = gbf ? 2 : 4, target = cfg.bucket_bytes > 0 ? (size_t)cfg.bucket_bytes : (size_t)25 << 20;
      if (!lay.tied) { Bucket b; b.off = lay.head; b.n = V * D; b.producers = {"head dW", "head dX"}; b.adam_phases = {"adamw head"}; b.last_layer = -1; buckets.push_back(b); }
      int hi = L - 1;
      while (hi >= 0) {
        int lo = hi;
        auto bytes = [&](int a, int z) { const size_t end = (z + 1 < L) ? lay.g1[z + 1] : lay.gf + D; return (end - lay.g1[a]) * esz; };
        while (lo > 0 && bytes(lo, hi) < target) lo--;
        Bucket b; b.off = lay.g1[lo]; b.n = ((hi + 1 < L) ? lay.g1[hi + 1] : lay.gf + D) - lay.g1[lo]; b.last_layer = lo;
        for (int l = lo; l <= hi; l++) { bucket_of_layer[l] = (int)buckets.size(); b.adam_phases.push_back("adamw L" + std::to_string(l)); }
        buckets.push_back(b);
        hi = lo - 1;
      }
      { Bucket b; b.off = lay.wte; b.n = V * D + (size_t)m.T * D; b.producers = {"embed bwd wte", "embed bwd wpe", "head dX"}; if (lay.tied) b.producers.push_back("head dW");
        b.adam_phases = {"adamw wte", "adamw wpe"}; b.last_layer = -2; buckets.push_back(b); }
      if (buckets.size() > 32) { c->err = "more than 32 gradient buckets"; return false; }
    }
    c->buckets.clear();
    for (const Bucket& b : buckets) c->buckets.push_back(Span{b.off, b.n});
    auto signal = [&](int bi) {
      PhaseDesc d = mk(TK_EXT_SIGNAL, 1); d.p[0] = c->d_ext_ready + bi;
      addp("grads ready " + std::to_string(bi), d, buckets[bi].producers, {});
    };

    // ---- optimizer helpers. Optionally (cfg.adam_interleave, and only without external gradient synchronisation) a layer's
    // AdamW is placed INSIDE the backward pass, one layer below the one it updates, instead of after it. Off by default: on the
    // full model it measured 0.5-0.9 % slower per step (the memory-bound tasks delay the chain of small backward phases).
    auto gate = [&](const std::string& adam_name, std::vector<std::string> deps) {
      if (!ext) return deps;
      for (size_t bi = 0; bi < buckets.size(); bi++) for (const std::string& a : buckets[bi].adam_phases) if (a == adam_name) return std::vector<std::string>{"allreduce done " + std::to_string(bi)};
      return deps;
    };
    auto mkadam = [&](size_t off, size_t n, const std::vector<Span>& nodecay) {
      PhaseDesc d = mk(TK_ADAMW, (int)((n + ew::OPT_CHUNK - 1) / ew::OPT_CHUNK));
      d.p[0] = c->W32 + off; d.p[1] = G(off); d.p[2] = c->M32 + off; d.p[3] = c->V32 + off; d.p[4] = Wact + off;
      d.n = n; d.i0 = (int)nodecay.size(); d.i1 = gbf ? 1 : 0;
      d.i2 = getenv("OFA_B200_ADAM_DIRECT") ? 1 : 0;     // A/B switch for measurements: 1 = the loop of direct loads instead of the staged inputs
      std::vector<int2> nd; for (const Span& sp : nodecay) nd.push_back(make_int2((int)(sp.off - off), (int)(sp.off - off + sp.n)));
      int2* dn = c->ar.alloc<int2>(std::max<size_t>(1, nd.size()));
      if (dn && !nd.empty()) c->ar.h2d(dn, nd.data(), nd.size() * sizeof(int2));
      d.p[5] = dn;
      return d;
    };
    auto emit_adam_head = [&]() { addp("adamw head", mkadam(lay.head, V * D, {}), gate("adamw head", {"head dW", "head dX"}), {}); };
    auto emit_adam_layer = [&](int l) {
      const std::string s = "L" + std::to_string(l) + " ";
      const size_t off = lay.g1[l], end = (l + 1 < L) ? lay.g1[l + 1] : lay.gf + D;
      std::vector<Span> nd = {Span{lay.g1[l], D}, Span{lay.g2[l], D}};
      std::vector<std::string> deps = {s + "dWdown", s + "dWup", s + "dgamma2", s + "dWo", s + "dWqkv", s + "dgamma1", s + "ln1 bwd"};
      if (l == L - 1) { nd.push_back(Span{lay.gf, D}); deps.push_back("lnf dgamma"); }
      addp("adamw L" + std::to_string(l), mkadam(off, end - off, nd), gate("adamw L" + std::to_string(l), deps), {});
    };
    const bool interleave_adam = train && !ext && cfg.adam_interleave == 1;
    // cfg.adam_interleave = n >= 2 (off by default: measured 0.9-1.5 % slower per step for n = 6..48, because an AdamW task is bound
    // by what one block keeps in flight - 88 us beside GEMMs against 100 us beside 231 others like it - so moving it buys little and
    // costs the chain its earliest blocks): AdamW trickles through the backward pass. As soon as a tensor group's gradient is final its
    // update is queued, and after every backward phase up to n optimizer tasks are emitted as a small phase of their own. A
    // backward phase of 192 strips leaves 40 of the 232 training blocks without a ticket; they take these tasks instead of
    // waiting, and a memory-bound task that runs beside GEMMs instead of beside 231 others like it finishes several times
    // sooner. The group's usual phase name goes to a 1-task phase behind its last chunk that waits for all of them, so the next
    // step's forward pass still has one thing to wait for.
    struct AdamItem { std::string name; size_t off, n; std::vector<Span> nd; std::vector<std::string> deps, parts; int next_task = 0, chunks = 0; };
    std::vector<AdamItem> adam_q; size_t adam_q_head = 0;
    const int trickle_n = (train && !ext && cfg.adam_interleave >= 2) ? cfg.adam_interleave : 0;
    bool in_trickle = false;
    auto mkadam_range = [&](size_t off, size_t n, const std::vector<Span>& nodecay_abs) {
      std::vector<Span> clipped;
      for (const Span& sp : nodecay_abs) {
        const size_t lo = std::max(sp.off, off), hi = std::min(sp.off + sp.n, off + n);
        if (lo < hi) clipped.push_back(Span{lo, hi - lo});
      }
      return mkadam(off, n, clipped);
    };
    auto trickle = [&](bool flush) {
      if (!trickle_n || in_trickle) return;
      in_trickle = true;
      long budget = flush ? (1L << 40) : trickle_n;
      while (budget > 0 && adam_q_head < adam_q.size()) {
        AdamItem& it = adam_q[adam_q_head];
        const int total = (int)((it.n + ew::OPT_CHUNK - 1) / ew::OPT_CHUNK);
        int cnt = (int)std::min<long>(budget, total - it.next_task);
        if (total - it.next_task - cnt < trickle_n / 2) cnt = total - it.next_task;        // no tiny remainder
        const bool last = it.next_task + cnt == total;
        const size_t o = it.off + (size_t)it.next_task * ew::OPT_CHUNK, nn = std::min((size_t)cnt * ew::OPT_CHUNK, it.off + it.n - o);
        if (last && it.chunks == 0) {                    // the whole group in one piece: an ordinary optimizer phase
          addp(it.name, mkadam_range(o, nn, it.nd), it.deps, {});
        } else {
          // chunks are independent of one another (a chain would serialise the group and park the blocks that hold the
          // later chunks' tickets); one 1-task phase in front says "the gradient is final", one behind says "all chunks done"
          if (it.chunks == 0) addp(it.name + " ready", mk(TK_BARRIER, 1), it.deps, {});
          const std::string nm = it.name + " ." + std::to_string(it.chunks);
          addp(nm, mkadam_range(o, nn, it.nd), {it.name + " ready"}, {});
          it.parts.push_back(nm);
          if (last) addp(it.name, mk(TK_BARRIER, 1), it.parts, {});
        }
        it.chunks++; it.next_task += cnt; budget -= cnt;
        if (last) adam_q_head++;
      }
      in_trickle = false;
    };
    auto addb = [&](const std::string& name, const PhaseDesc& d, std::vector<std::string> deps0, std::vector<std::string> deps_prev, std::vector<std::string> rbdeps = {}) {
      addp(name, d, deps0, deps_prev, rbdeps);
      trickle(false);
    };

    // ---- backward
    {
      // head dX has K = V: 192 tiles with a very long main loop (0.39 ms per tile). Optionally (cfg.head_dx_splitk) it is cut into
      // S partial products over disjoint K ranges (fp32 partials, fixed summation order). Off by default: on the full model
      // it measured 1.2 % slower per step, the long tiles run beside head dW and are not what the step waits for.
      int S = 1;
      if (bf && V >= 8192 && cfg.head_dx_splitk) for (int c = 4; c >= 2; c--) if (V % (64 * (size_t)c) == 0) { S = c; break; }
      if (S == 1) addp("head dX", mkgemm(GL_NN, GE_STORE, logits, V, Wact + lay.head, D, dxf, D, nullptr, 0, N, D, V, 0), {"cross-entropy"}, {}, {"cross-entropy"});
      else {
        const size_t Ks = V / S;
        std::vector<std::string> parts;
        PhaseDesc dsum = mk(TK_SUMCAST, (int)((N * D + ew::SUM_CHUNK - 1) / ew::SUM_CHUNK)); dsum.p[0] = dxf; dsum.i0 = S; dsum.n = N * D;
        for (int k = 0; k < S; k++) {
          float* part = abuf<float>(c, "dxf_part" + std::to_string(k), N * D);
          dsum.p[1 + k] = part;
          const std::string nm = "head dX k" + std::to_string(k);
          addp(nm, mkgemm(GL_NN, GE_F32, logits + k * Ks, V, Wact + lay.head + k * Ks * D, D, part, D, nullptr, 0, N, D, (int)Ks, 0), {"cross-entropy"}, {});
          parts.push_back(nm);
        }
        if (!c->ar.ok) { c->err = "out of device memory (split-K partials)"; return false; }
        addp("head dX", dsum, parts, {});
      }
    }
    addb("head dW", mkgemm(GL_TN, wepi, logits, V, lnf, D, G(lay.head), D, nullptr, 0, V, D, N, 0, /*wide=*/1), {"cross-entropy"}, {});
    if (trickle_n && !lay.tied) { AdamItem it; it.name = "adamw head"; it.off = lay.head; it.n = V * D; it.deps = {"head dW", "head dX"}; adam_q.push_back(it); }
    if (ext && !lay.tied) signal(0);
    { PhaseDesc d = mk(TK_LN_BWD, rows16); d.p[0] = dxs[L]; d.p[1] = dgpf; d.p[2] = dxf; d.p[3] = xs[L]; d.p[4] = meanf; d.p[5] = rstdf; d.p[6] = Wact + lay.gf; d.p[7] = nullptr;
      addb("lnf bwd", d, {"head dX"}, {}, {"head dX"}); }
    auto mkdg = [&](float* part, size_t goff) { PhaseDesc d = mk(TK_LN_DG, (int)((D + NTHR - 1) / NTHR)); d.p[0] = G(goff); d.p[1] = part; d.i0 = 0; d.i1 = gbf ? 1 : 0; return d; };
    addb("lnf dgamma", mkdg(dgpf, lay.gf), {"lnf bwd"}, {});
    std::string g = "lnf bwd";
    const int attn_bwd_tasks = bf ? 2 * attn_fwd_tasks : m.B * m.H;
    for (int l = L - 1; l >= 0; l--) {
      const std::string s = "L" + std::to_string(l) + " ";
      addb(s + "dpre", mkgemm(GL_NT, GE_DGELU, dxs[l + 1], D, Wact + lay.wdn[l], D, dpre[l], FF, upre[l], FF, N, FF, D, 0), {g}, {}, {g});
      addb(s + "dWdown", mkgemm(GL_TN, wepi, uact[l], FF, dxs[l + 1], D, G(lay.wdn[l]), D, nullptr, 0, FF, D, N, 0), {g}, {});
      if (interleave_adam) { if (l == L - 1) { if (!lay.tied) emit_adam_head(); } else emit_adam_layer(l + 1); }
      addb(s + "dln2", mkgemm(GL_NT, GE_STORE, dpre[l], FF, Wact + lay.wup[l], FF, dln2[l], D, nullptr, 0, N, D, FF, 0), {s + "dpre"}, {}, {s + "dpre"});
      addb(s + "dWup", mkgemm(GL_TN, wepi, ln2[l], D, dpre[l], FF, G(lay.wup[l]), FF, nullptr, 0, D, FF, N, 0), {s + "dpre"}, {});
      { PhaseDesc d = mk(TK_LN_BWD, rows16); d.p[0] = dh[l]; d.p[1] = dgp2[l]; d.p[2] = dln2[l]; d.p[3] = hb[l]; d.p[4] = mean2[l]; d.p[5] = rstd2[l]; d.p[6] = Wact + lay.g2[l]; d.p[7] = dxs[l + 1];
        addb(s + "ln2 bwd", d, {s + "dln2"}, {}, {s + "dln2"}); }
      addb(s + "dgamma2", mkdg(dgp2[l], lay.g2[l]), {s + "ln2 bwd"}, {});
      if (bf) {   // the epilogue also forms the row term of attention backward, D[b,h,t] = sum_d dO * O: no separate pass over dO and O
        PhaseDesc d = mkgemm(GL_NT, GE_DR, dh[l], D, Wact + lay.wo[l], D, dob[l], D, att[l], D, N, D, D, 0);
        d.g.dr = Dr[l]; d.g.dr_T = m.T; d.g.dr_H = m.H;
        addb(s + "dO", d, {s + "ln2 bwd"}, {}, {s + "ln2 bwd"});
      } else {
        addb(s + "dO", mkgemm(GL_NT, GE_STORE, dh[l], D, Wact + lay.wo[l], D, dob[l], D, nullptr, 0, N, D, D, 0), {s + "ln2 bwd"}, {});
      }
      addb(s + "dWo", mkgemm(GL_TN, wepi, att[l], D, dh[l], D, G(lay.wo[l]), D, nullptr, 0, D, D, N, 0), {s + "ln2 bwd"}, {});
      if (!bf) { PhaseDesc d = mk(TK_ATT_PREP, 1); d.p[0] = att[l]; d.p[1] = dob[l]; d.p[2] = Dr[l]; addb(s + "attn prep", d, {s + "dO"}, {}); }
      { PhaseDesc d = mk(TK_ATT_BWD, attn_bwd_tasks); d.p[0] = qkv[l]; d.p[1] = dob[l]; d.p[2] = lse[l]; d.p[3] = Dr[l]; d.p[4] = dqkv[l]; d.p[5] = att[l];
        if (bf) { std::string e; d.p[6] = const_cast<void*>(make_attn_maps(c->ar, qkv[l], dob[l], N, D, e)); if (!d.p[6]) { ok = false; err = e; } }
        addb(s + "attn bwd", d, {bf ? s + "dO" : s + "attn prep"}, {}, {s + "dO"}); }
      addb(s + "dln1", mkgemm(GL_NT, GE_STORE, dqkv[l], 3 * D, Wact + lay.wqkv[l], 3 * D, dln1[l], D, nullptr, 0, N, D, 3 * D, 0), {s + "attn bwd"}, {}, {s + "attn bwd"});
      addb(s + "dWqkv", mkgemm(GL_TN, wepi, ln1[l], D, dqkv[l], 3 * D, G(lay.wqkv[l]), 3 * D, nullptr, 0, D, 3 * D, N, 0), {s + "attn bwd"}, {});
      { PhaseDesc d = mk(TK_LN_BWD, rows16); d.p[0] = dxs[l]; d.p[1] = dgp1[l]; d.p[2] = dln1[l]; d.p[3] = xs[l]; d.p[4] = mean1[l]; d.p[5] = rstd1[l]; d.p[6] = Wact + lay.g1[l]; d.p[7] = dh[l];
        addb(s + "ln1 bwd", d, {s + "dln1"}, {}, {s + "dln1"}); }
      addb(s + "dgamma1", mkdg(dgp1[l], lay.g1[l]), {s + "ln1 bwd"}, {});
      g = s + "ln1 bwd";
      if (trickle_n) {
        AdamItem it; it.name = "adamw L" + std::to_string(l); it.off = lay.g1[l]; it.n = ((l + 1 < L) ? lay.g1[l + 1] : lay.gf + D) - lay.g1[l];
        it.nd = {Span{lay.g1[l], D}, Span{lay.g2[l], D}};
        it.deps = {s + "dWdown", s + "dWup", s + "dgamma2", s + "dWo", s + "dWqkv", s + "dgamma1", s + "ln1 bwd"};
        if (l == L - 1) { it.nd.push_back(Span{lay.gf, D}); it.deps.push_back("lnf dgamma"); }
        adam_q.push_back(it);
      }
      if (ext) {
        Bucket& b = buckets[bucket_of_layer[l]];
        for (const char* nm : {"dWdown", "dWup", "dgamma2", "dWo", "dWqkv", "dgamma1", "ln1 bwd"}) b.producers.push_back(s + nm);
        if (l == L - 1) b.producers.push_back("lnf dgamma");
        if (b.last_layer == l) signal(bucket_of_layer[l]);
      }
    }
    { PhaseDesc d = mk(TK_EMB_WTE, (int)((V + ew::EMB_VCHUNK - 1) / ew::EMB_VCHUNK)); d.p[0] = G(lay.wte); d.p[1] = dxs[0]; d.p[2] = c->C.tok_in; d.i0 = lay.tied ? 1 : 0; d.i1 = gbf ? 1 : 0;
      addp("embed bwd wte", d, {"L0 ln1 bwd", lay.tied ? "head dW" : ""}, {}); }
    { PhaseDesc d = mk(TK_EMB_WPE, (m.T + ew::WPE_ROWS - 1) / ew::WPE_ROWS); d.p[0] = G(lay.wpe); d.p[1] = dxs[0]; d.i1 = gbf ? 1 : 0; addp("embed bwd wpe", d, {"L0 ln1 bwd"}, {}); }
    if (ext) signal((int)buckets.size() - 1);
    end_deps = {"loss mean", "embed bwd wte", "embed bwd wpe", "head dW", "head dX", "lnf dgamma"};
    for (int l = 0; l < L; l++) { const std::string s = "L" + std::to_string(l) + " "; for (const char* nm : {"dWdown", "dWup", "dgamma2", "dWo", "dWqkv", "dgamma1"}) end_deps.push_back(s + nm); }
    if (train) {
      // ---- optimizer phases that were not already emitted inside the backward pass
      end_deps = {"loss mean"};
      if (ext) for (size_t bi = 0; bi < buckets.size(); bi++) {
        PhaseDesc d = mk(TK_EXT_WAIT, 1); d.p[0] = c->d_ext_done + bi;
        addp("allreduce done " + std::to_string(bi), d, {"grads ready " + std::to_string(bi)}, {});
      }
      trickle(true);                                   // what the backward pass had no room for
      if (!lay.tied && !id.count("adamw head")) emit_adam_head();
      for (int l = L - 1; l >= 0; l--) if (!id.count("adamw L" + std::to_string(l))) emit_adam_layer(l);
      if (!lay.tied) end_deps.push_back("adamw head");
      for (int l = 0; l < L; l++) end_deps.push_back("adamw L" + std::to_string(l));
      addp("adamw wte", mkadam(lay.wte, V * D, {}), gate("adamw wte", {"embed bwd wte", "head dX", lay.tied ? "head dW" : ""}), {});
      addp("adamw wpe", mkadam(lay.wpe, (size_t)m.T * D, {}), gate("adamw wpe", {"embed bwd wpe"}), {});
      end_deps.push_back("adamw wte"); end_deps.push_back("adamw wpe");
    }
  }
  { PhaseDesc d = mk(TK_BARRIER, 1); addp(step_end, d, end_deps, {}); }
  if (!ok) { c->err = err; return false; }
  if (!c->ar.ok) { c->err = "out of device memory (graph tables)"; return false; }
  for (size_t i = 0; i < P.size(); i++)
    for (const std::string& nm : prevdeps[i]) {
      auto it = id.find(nm);
      if (it == id.end()) { c->err = "unknown cross-step dependency " + nm + " of " + P[i].name; return false; }
      P[i].deps.push_back(Dep{it->second, -1});
    }
  c->train_last = id[step_end];
  return true;
}

// ---------------------------------------------------------------------------------------------- serving graph
template <class T>
bool build_decode_graph(ofa_ctx* c) {
  const ModelDims& m = c->md; const Layout& lay = c->lay; const ofa_config& cfg = c->cfg;
  const T* Wact = reinterpret_cast<const T*>(c->Wact);
  const int L = m.L, D = m.D;
  const int nchunk = (m.V + dec::HR - 1) / dec::HR;
  DecodeParams& dp = c->C.dp;
  memset(&dp, 0, sizeof dp);
  dp.wte = Wact + lay.wte; dp.wpe = Wact + lay.wpe; dp.head = Wact + lay.head; dp.gf = Wact + lay.gf;
  std::vector<const void*> hq(L), ho(L), hu(L), hd(L), h1(L), h2(L);
  for (int l = 0; l < L; l++) { hq[l] = Wact + lay.wqkv[l]; ho[l] = Wact + lay.wo[l]; hu[l] = Wact + lay.wup[l]; hd[l] = Wact + lay.wdn[l]; h1[l] = Wact + lay.g1[l]; h2[l] = Wact + lay.g2[l]; }
  auto up = [&](const std::vector<const void*>& h) { const void** d = c->ar.alloc<const void*>(L); if (d) c->ar.h2d(d, h.data(), L * sizeof(void*)); return (const void* const*)d; };
  dp.wqkv = up(hq); dp.wo = up(ho); dp.wup = up(hu); dp.wdn = up(hd); dp.g1 = up(h1); dp.g2 = up(h2);
  {  // unswizzled 2-D views for the weight prefetch: one 64-column (QKV) / 32-column (up) / head-by-column-block (Wo) box per copy
    const bool f32w = !c->bf;
    const uint32_t brow = D < 256 ? D : 256, cbw = D < 256 ? D : 256;
    std::vector<CUtensorMap> mq(L), mu(L), mo(L);
    bool okm = true;
    for (int l = 0; l < L && !c->ar.dry; l++) {
      okm = okm && encode_map(&mq[l], hq[l], 3 * D, D, 3 * D, 64, brow, f32w, false) && encode_map(&mu[l], hu[l], m.FF, D, m.FF, dec::HU, brow, f32w, false) &&
            encode_map(&mo[l], ho[l], D, D, D, cbw, m.DH, f32w, false);
    }
    if (!okm) { c->err = "cuTensorMapEncodeTiled failed (decode prefetch views)"; return false; }
    CUtensorMap* dq = c->ar.alloc<CUtensorMap>(L, false); CUtensorMap* du = c->ar.alloc<CUtensorMap>(L, false); CUtensorMap* dw = c->ar.alloc<CUtensorMap>(L, false);
    if (dq && du && dw) { c->ar.h2d(dq, mq.data(), L * sizeof(CUtensorMap)); c->ar.h2d(du, mu.data(), L * sizeof(CUtensorMap)); c->ar.h2d(dw, mo.data(), L * sizeof(CUtensorMap)); }
    dp.tm_qkv = dq; dp.tm_up = du; dp.tm_wo = dw;
  }
  DecodeState& st = dp.st;
  st.xw = c->ar.alloc<unsigned long long>(D); st.xr = c->ar.alloc<unsigned long long>(D);
  st.q = c->ar.alloc<T>(D);
  st.cand_v = c->ar.alloc<float>(2 * nchunk); st.cand_i = c->ar.alloc<int>(2 * nchunk);
  c->d_scal = c->ar.alloc<int>(8); st.scal = c->d_scal;
  st.kv = c->ar.alloc<T>((size_t)L * 2 * m.H * m.T * m.DH);
  st.logits = c->ar.alloc<float>(m.V);
  c->bufs["dec_kv"] = std::make_pair((void*)st.kv, (size_t)L * 2 * m.H * m.T * m.DH * sizeof(T));   // [L][2][H][T][DH], for parity checks
  c->bufs["dec_scal"] = std::make_pair((void*)c->d_scal, sizeof(int) * 8);                               // token, pos, step, ctx_full, astep, poskey, epoch
  c->out_cap = cfg.decode_out_cap > 0 ? cfg.decode_out_cap : 65536;
  if (c->ar.dry) { c->d_out = c->ar.alloc<int>(c->out_cap); }
  else {
    if (cudaHostAlloc(&c->h_out, sizeof(int) * c->out_cap, cudaHostAllocMapped) != cudaSuccess) { c->err = "cudaHostAlloc failed"; return false; }
    memset(c->h_out, 0xFF, sizeof(int) * c->out_cap);
    cudaHostGetDevicePointer(&c->d_out, c->h_out, 0);
  }
  st.out_tokens = c->d_out; st.out_cap = c->out_cap;
  c->d_forced = c->ar.alloc<int>(std::max(1, cfg.n_prompt));
  dp.trace = c->ar.alloc<unsigned long long>(64);
  if (!c->ar.ok) { c->err = "out of device memory (decode state)"; return false; }
  c->ar.h2d(c->d_forced, cfg.prompt, sizeof(int) * cfg.n_prompt);
  dp.forced = c->d_forced; dp.nforced = cfg.n_prompt; dp.answer_len = cfg.answer_len; dp.auto_reset = 1;
  dp.temperature = cfg.temperature; dp.seed = cfg.decode_seed;
  int scal[8] = {cfg.prompt[0], 0, 0, 0, 0, 0, 0, 0};
  c->ar.h2d(c->d_scal, scal, sizeof scal);

  std::vector<HostPhase>& P = c->dec_ph; P.clear();
  auto mk = [&](const std::string& name, int kind, int ntasks, int layer) {
    HostPhase hp; hp.name = name; memset(&hp.d, 0, sizeof hp.d); hp.d.kind = kind; hp.d.ntasks = ntasks; hp.d.i0 = layer;
    if (!P.empty()) hp.deps.push_back(Dep{(int)P.size() - 1, 0});
    P.push_back(hp);
  };
  const int CB = D < 256 ? D : 256;
  for (int l = 0; l < L; l++) {
    const std::string s = "dec L" + std::to_string(l) + " ";
    mk(s + "qkv", TK_DEC_QKV, 3 * D / 64, l);
    mk(s + "att+wo", TK_DEC_ATTWO, m.H * (D / CB), l);
    mk(s + "up+down", TK_DEC_UPDN, m.FF / dec::HU, l);
  }
  mk("dec head", TK_DEC_HEAD, nchunk, 0);
  mk("dec sample", TK_DEC_SAMPLE, 1, 0);
  P[0].deps.push_back(Dep{(int)P.size() - 1, -1});
  c->dec_last = (int)P.size() - 1;
  return true;
}

bool probe_smids(ofa_ctx* c) {
  unsigned* seen = c->ar.alloc<unsigned>(64);
  if (!seen) return false;
  cudaFuncSetAttribute(smid_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, c->smem);
  cudaFuncSetAttribute(smid_probe_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  smid_probe_kernel<<<c->nblocks, NTHR, c->smem, c->stream>>>(seen);
  if (cudaStreamSynchronize(c->stream) != cudaSuccess) return false;
  unsigned h[64]; cudaMemcpy(h, seen, sizeof h, cudaMemcpyDeviceToHost);
  std::vector<int> rank(2048, -1); int n = 0; bool dense = true;
  for (int i = 0; i < 2048; i++) if (h[i >> 5] >> (i & 31) & 1u) { if (i != n) dense = false; rank[i] = n++; }
  if (n == 0) return false;
  if (!dense || n != c->num_sms) {
    for (int i = 0; i < 2048; i++) if (rank[i] < 0) rank[i] = 1 << 20;   // unknown SM: idle
    c->d_smid_rank = c->ar.alloc<int>(2048);
    if (!c->d_smid_rank) return false;
    cudaMemcpy(c->d_smid_rank, rank.data(), 2048 * sizeof(int), cudaMemcpyHostToDevice);
  }
  return true;
}

int read_f32(ofa_ctx* c, const float* src, float* out, size_t n) {
  if (c && c->dry) return fail(c, OFA_BAD_ARGUMENT, "planning context (device < 0) has no device memory");
  if (!c || !out || n > c->lay.total) return fail(c, OFA_BAD_ARGUMENT, "bad size");
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "launch in flight: call ofa_wait first");
  return cudaMemcpy(out, src, n * sizeof(float), cudaMemcpyDeviceToHost) == cudaSuccess ? OFA_OK : fail(c, OFA_CUDA_ERROR, cudaGetErrorString(cudaGetLastError()));
}

__global__ void f32_to_act_kernel(const float* src, bf16* dst, size_t n) { for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = __float2bfloat16(src[i]); }
__global__ void f32_to_act_kernel(const float* src, float* dst, size_t n) { for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = src[i]; }
__global__ void bf16_to_f32_kernel(const bf16* src, float* dst, size_t n) { for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = __bfloat162float(src[i]); }

}  // namespace

// ================================================================================================ C ABI: model level
extern "C" int ofa_default_config(ofa_config* cfg, const char* preset) {
  if (!cfg || !preset) return OFA_BAD_ARGUMENT;
  memset(cfg, 0, sizeof *cfg);
  cfg->beta1 = 0.9f; cfg->beta2 = 0.95f; cfg->eps = 1e-8f; cfg->weight_decay = 0.1f;
  cfg->sched_profile = 1;
  cfg->dp_world = 1; cfg->temperature = 0.f; cfg->decode_seed = 1234; cfg->data_seed = 0; cfg->decode_out_cap = 65536;
  if (!strcmp(preset, "tiny")) {
    cfg->vocab = 65; cfg->d_model = 64; cfg->n_layer = 2; cfg->n_head = 4; cfg->ctx_len = 64; cfg->batch = 16; cfg->valid_vocab = 65;
    cfg->dtype = OFA_DTYPE_F32; cfg->constant_lr = 1; cfg->lr_max = 3e-4f; cfg->lr_min = 3e-4f; cfg->warmup = 0; cfg->sched_steps = 1;
    cfg->answer_len = 64; cfg->n_prompt = 8;
  } else if (!strcmp(preset, "gpt_s")) {
    cfg->vocab = 50304; cfg->d_model = 768; cfg->n_layer = 12; cfg->n_head = 12; cfg->ctx_len = 1024; cfg->batch = 4; cfg->valid_vocab = 50304;
    cfg->dtype = OFA_DTYPE_BF16; cfg->lr_max = 6e-4f; cfg->lr_min = 6e-5f; cfg->warmup = 100; cfg->sched_steps = 4000;
    cfg->answer_len = 256; cfg->n_prompt = 6;
  } else return OFA_BAD_ARGUMENT;
  return OFA_OK;
}

extern "C" const char* ofa_last_error(const ofa_ctx* ctx) { return ctx ? ctx->err.c_str() : g_create_error.c_str(); }

// Host-requested abort: raises the grid-wide abort word; every bounded wait on the device sees it and the kernel returns.
static void post_abort(ofa_ctx* c) {
  static const int one = 1;
  if (!c->abort_stream) cudaStreamCreateWithFlags(&c->abort_stream, cudaStreamNonBlocking);
  cudaMemcpyAsync(&c->d_status->abort, &one, sizeof(int), cudaMemcpyHostToDevice, c->abort_stream);
}
extern "C" int ofa_abort(ofa_ctx* c) {
  if (!c || c->dry) return OFA_BAD_ARGUMENT;
  if (!c->in_flight) return OFA_NOT_LAUNCHED;
  cudaSetDevice(c->device);
  c->abort_requested = true;
  post_abort(c);
  return OFA_OK;
}

extern "C" void ofa_destroy(ofa_ctx* c) {
  if (!c) return;
  if (c->dry) { delete c; return; }
  cudaSetDevice(c->device);
  if (c->in_flight) {
    // never block forever: ask the kernel to drain, give it a few seconds, and otherwise leak the device memory it may still use
    ofa_abort(c);
    bool done = false;
    for (int i = 0; i < 25000 && !done; i++) { done = cudaEventQuery(c->ev1) != cudaErrorNotReady; if (!done) { if (i % 64 == 63) post_abort(c); struct timespec sl = {0, 200000}; nanosleep(&sl, nullptr); } }
    if (!done) { delete c; return; }
  }
  ofa_dp_shutdown(c);
  c->train_job.free_all(); c->dec_job.free_all();
  if (c->d_step_done) cudaFree(c->d_step_done);
  if (c->d_tokens) cudaFree(c->d_tokens);
  if (c->d_starts) cudaFree(c->d_starts);
  c->ar.free_all();
  if (c->h_live) cudaFreeHost(c->h_live);
  if (c->h_out) cudaFreeHost(c->h_out);
  if (c->ev0) cudaEventDestroy(c->ev0);
  if (c->ev1) cudaEventDestroy(c->ev1);
  if (c->stream) cudaStreamDestroy(c->stream);
  if (c->abort_stream) cudaStreamDestroy(c->abort_stream);
  delete c;
}

extern "C" int ofa_create(const ofa_config* cfg, ofa_ctx** out) {
  if (!cfg || !out) return fail(nullptr, OFA_BAD_ARGUMENT, "null argument");
  *out = nullptr;
  ofa_ctx* c = new ofa_ctx();
  auto bail = [&](int code, const std::string& msg) { g_create_error = msg; ofa_destroy(c); return code; };
  c->cfg = *cfg;
  ModelDims& m = c->md;
  m.V = cfg->vocab; m.D = cfg->d_model; m.L = cfg->n_layer; m.H = cfg->n_head; m.T = cfg->ctx_len; m.B = cfg->batch;
  m.N = m.B * m.T; m.FF = 4 * m.D; m.DH = m.H > 0 ? m.D / m.H : 0; m.valid_vocab = cfg->valid_vocab > 0 ? cfg->valid_vocab : m.V;
  c->bf = cfg->dtype == OFA_DTYPE_BF16;
  if (m.V <= 0 || m.L <= 0 || m.H <= 0 || m.T <= 0 || m.B <= 0 || m.L > 64) return bail(OFA_BAD_CONFIG, "non-positive model dimension");
  if (c->bf) {
    if (m.D != 768 || m.DH != 64) return bail(OFA_BAD_CONFIG, "bf16 path is built for d_model 768 / head_dim 64");
    if (m.V % 128 || m.N % 128 || m.T % 128) return bail(OFA_BAD_CONFIG, "bf16 path needs vocab, batch*ctx_len and ctx_len to be multiples of 128");
  } else {
    if (cfg->dtype != OFA_DTYPE_F32 || m.D != 64 || m.DH != 16) return bail(OFA_BAD_CONFIG, "fp32 path is built for d_model 64 / head_dim 16");
    if (m.T > 96) return bail(OFA_BAD_CONFIG, "fp32 attention keeps T x T scores in shared memory: ctx_len <= 96");
    if (cfg->grad_bf16) return bail(OFA_BAD_CONFIG, "grad_bf16 needs the bf16 path");
  }
  if (cfg->use_decode && (cfg->n_prompt < 1 || cfg->n_prompt > 32)) return bail(OFA_BAD_CONFIG, "decode needs 1..32 prompt tokens");
  if (cfg->use_decode && cfg->n_prompt > m.T) return bail(OFA_BAD_CONFIG, "prompt longer than ctx_len");
  for (int i = 0; i < cfg->n_prompt && cfg->use_decode; i++) if (cfg->prompt[i] < 0 || cfg->prompt[i] >= m.V) return bail(OFA_BAD_CONFIG, "prompt token out of range");
  if (cfg->mode < 0 || cfg->mode > 3) return bail(OFA_BAD_CONFIG, "bad mode");
  if (cfg->mode == OFA_MODE_DECODE_ONLY && !cfg->use_decode) return bail(OFA_BAD_CONFIG, "decode-only mode needs use_decode");
  if (cfg->dp_world < 1) return bail(OFA_BAD_CONFIG, "dp_world < 1");
  if (cfg->attn_legacy) return bail(OFA_BAD_CONFIG, "attn_legacy: the mma.sync attention tasks are no longer part of the library");

  c->device = cfg->device;
  const bool dry = cfg->device < 0;      // planning mode: build layout, buckets and phase graphs without touching a device
  c->ar.dry = dry; c->dry = dry;
  if (dry) { c->num_sms = 148; }
  else {
    if (cudaSetDevice(c->device) != cudaSuccess) return bail(OFA_CUDA_ERROR, "cudaSetDevice failed (no CUDA device?)");
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, c->device) != cudaSuccess) return bail(OFA_CUDA_ERROR, "cudaGetDeviceProperties failed");
    if (prop.major != 10) return bail(OFA_CUDA_ERROR, "this library contains sm_100a code only; device is sm_" + std::to_string(prop.major * 10 + prop.minor));
    c->num_sms = prop.multiProcessorCount;
  }
  c->nblocks = 2 * c->num_sms;
  c->smem = smem_for(c->bf, m.T, m.N);
  {
    const std::string e = smem_fit_error(c->bf, m.T, m.N, cfg->mode != OFA_MODE_FORWARD && cfg->mode != OFA_MODE_DECODE_ONLY, cfg->use_decode != 0, c->smem);
    if (!e.empty()) return bail(OFA_BAD_CONFIG, e);
  }
  if (!dry) {
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) return bail(OFA_CUDA_ERROR, "stream");
    cudaEventCreate(&c->ev0); cudaEventCreate(&c->ev1);
  }
  // SM split
  int infer = cfg->use_decode ? std::max(0, cfg->infer_sms) : 0, resv = std::max(0, cfg->reserved_sms);
  if (cfg->use_decode && infer == 0) infer = c->num_sms >= 148 ? 24 : std::max(1, c->num_sms / 6);
  const bool decode_only = cfg->mode == OFA_MODE_DECODE_ONLY;
  if (decode_only && cfg->infer_sms <= 0) infer = c->num_sms - resv;
  int train = decode_only ? 0 : (cfg->train_sms > 0 ? cfg->train_sms : c->num_sms - infer - resv);
  if (!decode_only && train <= 0) return bail(OFA_BAD_CONFIG, "no SMs left for the training job");
  if (infer + resv + train > c->num_sms || train < 0) return bail(OFA_BAD_CONFIG, "SM split exceeds the device's SM count");

  c->lay.build(m, cfg->tied_head != 0);
  const size_t NP = c->lay.total;
  c->W32 = c->ar.alloc<float>(NP); c->M32 = c->ar.alloc<float>(NP); c->V32 = c->ar.alloc<float>(NP);
  c->Wact = c->bf ? (void*)c->ar.alloc<bf16>(NP) : (void*)c->ar.alloc<float>(NP);
  if (cfg->grad_bf16) c->Gbf = c->ar.alloc<bf16>(NP); else c->G32 = c->ar.alloc<float>(NP);
  c->d_status = c->ar.alloc<DevStatus>(1); c->d_finished = c->ar.alloc<int>(2); c->d_t_end = c->ar.alloc<unsigned long long>(1);
  if (!c->ar.ok) return bail(OFA_CUDA_ERROR, "out of device memory (parameters)");
  if (!dry) {
    if (cudaHostAlloc(&c->h_live, sizeof(Live), cudaHostAllocMapped) != cudaSuccess) return bail(OFA_CUDA_ERROR, "cudaHostAlloc failed");
    memset(c->h_live, 0, sizeof(Live)); cudaHostGetDevicePointer(&c->d_live, c->h_live, 0);
  }
  c->d_ext_ready = c->ar.alloc<int>(64); c->d_ext_done = c->d_ext_ready ? c->d_ext_ready + 32 : nullptr;
  if (!c->ar.ok) return bail(OFA_CUDA_ERROR, "out of device memory");
  if (!dry && !probe_smids(c)) return bail(OFA_CUDA_ERROR, std::string("SM probe launch failed: ") + cudaGetErrorString(cudaGetLastError()));

  Ctx& C = c->C;
  memset(&C, 0, sizeof C);
  C.md = m;
  C.hp.lr_max = cfg->lr_max; C.hp.lr_min = cfg->lr_min; C.hp.beta1 = cfg->beta1; C.hp.beta2 = cfg->beta2; C.hp.eps = cfg->eps; C.hp.wd = cfg->weight_decay;
  C.hp.warmup = cfg->warmup; C.hp.sched_steps = std::max(cfg->sched_steps, cfg->warmup + 1); C.hp.constant_lr = cfg->constant_lr; C.hp.grad_scale = 1.0f / (float)cfg->dp_world;
  C.seed = cfg->data_seed;
  C.infer_sms = infer; C.reserved_sms = resv; C.train_sms = train; C.use_decode = cfg->use_decode ? 1 : 0; C.use_train = 1;
  C.smid_rank = c->d_smid_rank; C.live = c->d_live; C.status = c->d_status; C.finished = c->d_finished; C.t_end = c->d_t_end;
  C.dep_timeout_ns = (unsigned long long)((cfg->timeout_s > 0 ? cfg->timeout_s : 20.0) * 1e9);
  C.prof_step = -1;
  bool ok = decode_only ? true : (c->bf ? build_train_graph<bf16>(c) : build_train_graph<float>(c));
  if (!ok) return bail(OFA_BAD_CONFIG, "training graph: " + c->err);
  if (cfg->use_decode) {
    ok = c->bf ? build_decode_graph<bf16>(c) : build_decode_graph<float>(c);
    if (!ok) return bail(OFA_BAD_CONFIG, "decode graph: " + c->err);
  }
  const int nph = std::max<int>(1, (int)c->train_ph.size());
  c->d_phase_busy = c->ar.alloc<unsigned long long>(2 * nph);   /* busy, then dependency wait */ c->d_phase_first = c->ar.alloc<unsigned long long>(nph); c->d_phase_last = c->ar.alloc<unsigned long long>(nph);
  c->d_blk_busy = c->ar.alloc<unsigned long long>(6 * c->nblocks);
  if (!c->ar.ok) return bail(OFA_CUDA_ERROR, "out of device memory");
  c->d_dec_phase_busy = c->ar.alloc<unsigned long long>(std::max<size_t>(1, c->dec_ph.size()));
  c->d_blk_info = c->ar.alloc<int>(c->nblocks); C.blk_info = c->d_blk_info;
  C.phase_busy = c->d_phase_busy; C.phase_first = c->d_phase_first; C.phase_last = c->d_phase_last; C.blk_busy = c->d_blk_busy; C.blk_wait = c->d_blk_busy + 2 * c->nblocks; C.dec_phase_busy = c->d_dec_phase_busy;
  *out = c;
  return OFA_OK;
}

extern "C" size_t ofa_num_params(const ofa_ctx* c) { return c ? c->lay.total : 0; }
extern "C" int ofa_param_span(const ofa_ctx* c, const char* name, size_t* offset, size_t* count) {
  if (!c || !name) return OFA_BAD_ARGUMENT;
  auto it = c->lay.spans.find(name);
  if (it == c->lay.spans.end()) return OFA_BAD_ARGUMENT;
  if (offset) *offset = it->second.off;
  if (count) *count = it->second.n;
  return OFA_OK;
}

extern "C" int ofa_load_weights(ofa_ctx* c, const float* flat, size_t n) {
  if (c && c->dry) return fail(c, OFA_BAD_ARGUMENT, "planning context (device < 0) has no device memory");
  if (!c || !flat || n != c->lay.total) return fail(c, OFA_BAD_ARGUMENT, "weight count does not match the layout");
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "launch in flight");
  cudaSetDevice(c->device);
  if (cudaMemcpy(c->W32, flat, n * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) return fail(c, OFA_CUDA_ERROR, "H2D failed");
  if (c->bf) f32_to_act_kernel<<<1024, 256>>>(c->W32, reinterpret_cast<bf16*>(c->Wact), n);
  else f32_to_act_kernel<<<1024, 256>>>(c->W32, reinterpret_cast<float*>(c->Wact), n);
  cudaMemset(c->M32, 0, n * sizeof(float)); cudaMemset(c->V32, 0, n * sizeof(float));
  if (cudaDeviceSynchronize() != cudaSuccess) return fail(c, OFA_CUDA_ERROR, cudaGetErrorString(cudaGetLastError()));
  if (c->cfg.use_decode) {   // (re)start the decode context from the prompt with the new weights
    int scal[8] = {c->cfg.prompt[0], 0, 0, 0, 0, 0, 0, 0};
    cudaMemcpy(c->d_scal, scal, sizeof scal, cudaMemcpyHostToDevice);
    if (c->bf) decode_init_embed_kernel<bf16, 768><<<1, NTHR>>>(c->C.dp); else decode_init_embed_kernel<float, 64><<<1, NTHR>>>(c->C.dp);
    if (cudaDeviceSynchronize() != cudaSuccess) return fail(c, OFA_CUDA_ERROR, cudaGetErrorString(cudaGetLastError()));
    c->dec_steps_total = 0;
  }
  return OFA_OK;
}
extern "C" int ofa_read_weights(ofa_ctx* c, float* out, size_t n) { return c ? read_f32(c, c->W32, out, n) : OFA_BAD_ARGUMENT; }
extern "C" int ofa_read_adam_m(ofa_ctx* c, float* out, size_t n) { return c ? read_f32(c, c->M32, out, n) : OFA_BAD_ARGUMENT; }
extern "C" int ofa_read_adam_v(ofa_ctx* c, float* out, size_t n) { return c ? read_f32(c, c->V32, out, n) : OFA_BAD_ARGUMENT; }
extern "C" int ofa_read_grads(ofa_ctx* c, float* out, size_t n) {
  if (!c) return OFA_BAD_ARGUMENT;
  if (!c->cfg.grad_bf16) return read_f32(c, c->G32, out, n);
  if (c->dry) return fail(c, OFA_BAD_ARGUMENT, "planning context (device < 0) has no device memory");
  if (!out || n > c->lay.total) return fail(c, OFA_BAD_ARGUMENT, "bad size");
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "launch in flight: call ofa_wait first");
  cudaSetDevice(c->device);
  float* tmp = nullptr;
  if (cudaMalloc(&tmp, n * sizeof(float)) != cudaSuccess) return fail(c, OFA_CUDA_ERROR, "cudaMalloc failed");
  bf16_to_f32_kernel<<<1024, 256>>>(c->Gbf, tmp, n);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaMemcpy(out, tmp, n * sizeof(float), cudaMemcpyDeviceToHost);
  cudaFree(tmp);
  return e == cudaSuccess ? OFA_OK : fail(c, OFA_CUDA_ERROR, cudaGetErrorString(e));
}
extern "C" int ofa_load_adam_state(ofa_ctx* c, const float* mm, const float* vv, size_t n, int step_base) {
  if (c && c->dry) return fail(c, OFA_BAD_ARGUMENT, "planning context (device < 0) has no device memory");
  if (!c || !mm || !vv || n != c->lay.total || step_base < 0) return fail(c, OFA_BAD_ARGUMENT, "bad optimizer state");
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "launch in flight");
  cudaSetDevice(c->device);
  if (cudaMemcpy(c->M32, mm, n * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess || cudaMemcpy(c->V32, vv, n * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess)
    return fail(c, OFA_CUDA_ERROR, std::string("H2D failed: ") + cudaGetErrorString(cudaGetLastError()));
  c->steps_total = step_base;
  return OFA_OK;
}

extern "C" int ofa_set_tokens(ofa_ctx* c, const uint32_t* tokens, size_t n) {
  if (c && c->dry) return fail(c, OFA_BAD_ARGUMENT, "planning context (device < 0) has no device memory");
  if (!c || !tokens || n < (size_t)c->md.T + 2) return fail(c, OFA_BAD_ARGUMENT, "need more than ctx_len + 1 tokens");
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "launch in flight");
  for (size_t i = 0; i < n; i++) if (tokens[i] >= (uint32_t)c->md.V) return fail(c, OFA_BAD_ARGUMENT, "token id out of range");
  cudaSetDevice(c->device);
  if (n > c->tokens_cap) {                          // one buffer, grown when needed (the old one is freed)
    if (c->d_tokens) cudaFree(c->d_tokens);
    c->d_tokens = nullptr; c->tokens_cap = 0; c->ntok = 0;
    if (cudaMalloc(&c->d_tokens, n * 4) != cudaSuccess) return fail(c, OFA_CUDA_ERROR, "out of device memory");
    c->tokens_cap = n;
  }
  c->ntok = n;
  c->nstarts = 0;                                   // a starts table was validated against the old stream: it has to be set again
  return cudaMemcpy(c->d_tokens, tokens, n * 4, cudaMemcpyHostToDevice) == cudaSuccess ? OFA_OK : fail(c, OFA_CUDA_ERROR, "H2D failed");
}
extern "C" int ofa_set_starts(ofa_ctx* c, const uint32_t* starts, size_t nsteps) {
  if (!c) return OFA_BAD_ARGUMENT;
  if (c->dry) return fail(c, OFA_BAD_ARGUMENT, "planning context (device < 0) has no device memory");
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "launch in flight");
  if (!starts || nsteps == 0) { c->nstarts = 0; return OFA_OK; }
  const size_t n = nsteps * c->md.B;
  for (size_t i = 0; i < n; i++) if ((size_t)starts[i] + c->md.T + 1 > c->ntok) return fail(c, OFA_BAD_ARGUMENT, "start offset beyond the token stream (set tokens first)");
  cudaSetDevice(c->device);
  if (n > c->starts_cap) {
    if (c->d_starts) cudaFree(c->d_starts);
    c->d_starts = nullptr; c->starts_cap = 0; c->nstarts = 0;
    if (cudaMalloc(&c->d_starts, n * 4) != cudaSuccess) return fail(c, OFA_CUDA_ERROR, "out of device memory");
    c->starts_cap = n;
  }
  c->nstarts = (int)nsteps;
  return cudaMemcpy(c->d_starts, starts, n * 4, cudaMemcpyHostToDevice) == cudaSuccess ? OFA_OK : fail(c, OFA_CUDA_ERROR, "H2D failed");
}

extern "C" int ofa_launch(ofa_ctx* c, int nsteps) {
  if (c && c->dry) return fail(c, OFA_BAD_ARGUMENT, "planning context (device < 0) cannot launch");
  if (!c || nsteps <= 0) return fail(c, OFA_BAD_ARGUMENT, "nsteps must be positive");
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "previous launch still in flight: call ofa_wait");
  const bool train_on = c->C.train_sms > 0;
  if (train_on && (!c->d_tokens || c->ntok < (size_t)c->md.T + 2)) return fail(c, OFA_BAD_ARGUMENT, "no tokens set");
  cudaSetDevice(c->device);
  std::string err;
  if (train_on) {
    if (!upload_job(c->train_ph, c->train_last, nsteps, c->train_job, err, (c->bf && c->md.N % 128 == 0) ? c->md.N / 128 : 0)) return fail(c, OFA_BAD_CONFIG, err);
    if (c->steps_total + nsteps > c->loss_cap) {
      const int cap = std::max(4096, 2 * (c->steps_total + nsteps));
      float* nl = c->ar.alloc<float>(cap);
      if (!nl) return fail(c, OFA_CUDA_ERROR, "out of device memory");
      if (c->d_loss_hist) cudaMemcpy(nl, c->d_loss_hist, sizeof(float) * c->loss_cap, cudaMemcpyDeviceToDevice);
      c->d_loss_hist = nl; c->loss_cap = cap;
    }
    if (nsteps > c->step_done_cap) {               // grown, never re-allocated per launch: a loop of short launches must not leak
      if (c->d_step_done) cudaFree(c->d_step_done);
      c->d_step_done = nullptr; c->step_done_cap = 0;
      const int cap = std::max(1024, 2 * nsteps);
      if (cudaMalloc(&c->d_step_done, sizeof(unsigned long long) * cap) != cudaSuccess) return fail(c, OFA_CUDA_ERROR, "out of device memory");
      c->step_done_cap = cap;
    }
  }
  if (c->cfg.use_decode) {
    const int dsteps = train_on ? (1 << 20) : nsteps;
    if (!upload_job(c->dec_ph, c->dec_last, dsteps, c->dec_job, err)) return fail(c, OFA_BAD_CONFIG, err);
  }
  Ctx C = c->C;
  C.use_train = train_on ? 1 : 0;
  if (train_on) C.train = c->train_job.j;
  if (c->cfg.use_decode) C.dec = c->dec_job.j;
  fill_param_records(C, train_on ? &c->train_job : nullptr, c->cfg.use_decode ? &c->dec_job : nullptr);
  if (c->cfg.sched_profile) C.sched_flags |= 2;
  C.data = c->d_tokens; C.ntok = c->ntok; C.starts = c->nstarts > 0 ? c->d_starts : nullptr; C.nstarts = c->nstarts;
  C.loss_hist = c->d_loss_hist ? c->d_loss_hist + c->steps_total : nullptr;   // history, LR schedule and data windows continue across launches
  C.step_done = c->d_step_done;
  C.step_base = c->steps_total;
  c->abort_requested = false;
  cudaMemsetAsync(c->d_status, 0, sizeof(DevStatus), c->stream);
  cudaMemsetAsync(c->d_finished, 0, 2 * sizeof(int), c->stream);
  if (c->cfg.use_decode) {
    // The serving blocks of the previous launch left when training finished, normally in the middle of a token: the residual then
    // holds the contributions of some layers. The token is decoded again from layer 0 (the serving job's counters restart), so the
    // residual is rebuilt from the token and position the last completed sample step stored; K/V rows, q and candidates are rewritten.
    if (c->bf) decode_init_embed_kernel<bf16, 768><<<1, NTHR, 0, c->stream>>>(c->C.dp); else decode_init_embed_kernel<float, 64><<<1, NTHR, 0, c->stream>>>(c->C.dp);
  }
  C.arrived = c->d_finished + 1;
  cudaMemsetAsync(c->d_phase_busy, 0, sizeof(unsigned long long) * 2 * std::max<size_t>(1, c->train_ph.size()), c->stream);
  cudaMemsetAsync(c->d_blk_busy, 0, sizeof(unsigned long long) * 6 * c->nblocks, c->stream);
  cudaMemsetAsync(c->d_dec_phase_busy, 0, sizeof(unsigned long long) * std::max<size_t>(1, c->dec_ph.size()), c->stream);
  C.smem_bytes = c->smem;
  // wall-clock window of every phase in the last step of this launch (the reference's "phase wall-clock at step" table, ofa.cu:735-743)
  C.prof_step = nsteps - 1;
  cudaMemsetAsync(c->d_phase_first, 0xFF, sizeof(unsigned long long) * std::max<size_t>(1, c->train_ph.size()), c->stream);
  cudaMemsetAsync(c->d_phase_last, 0, sizeof(unsigned long long) * std::max<size_t>(1, c->train_ph.size()), c->stream);
  const Ctx& L = C;
  cudaEventRecord(c->ev0, c->stream);
  cudaError_t e = c->bf ? launch_kernel<bf16, 768, 64>(L, c->nblocks, c->smem, c->stream) : launch_kernel<float, 64, 16>(L, c->nblocks, c->smem, c->stream);
  cudaEventRecord(c->ev1, c->stream);
  if (e != cudaSuccess) return fail(c, OFA_CUDA_ERROR, std::string("kernel launch failed: ") + cudaGetErrorString(e));
  c->in_flight = true; c->last_nsteps = nsteps;
  return OFA_OK;
}

extern "C" int ofa_wait(ofa_ctx* c, int timeout_ms, ofa_status_t* status) {
  if (status) memset(status, 0, sizeof *status);
  if (!c) return OFA_BAD_ARGUMENT;
  if (!c->in_flight) { if (status) status->code = OFA_NOT_LAUNCHED; return fail(c, OFA_NOT_LAUNCHED, "nothing in flight"); }
  cudaSetDevice(c->device);
  struct timespec ts0; clock_gettime(CLOCK_MONOTONIC, &ts0);
  unsigned polls = 0;
  for (;;) {
    cudaError_t q = cudaEventQuery(c->ev1);
    if (q == cudaSuccess) break;
    if (q != cudaErrorNotReady) { c->in_flight = false; if (status) status->code = OFA_CUDA_ERROR; return fail(c, OFA_CUDA_ERROR, std::string("device error: ") + cudaGetErrorString(q)); }
    struct timespec ts; clock_gettime(CLOCK_MONOTONIC, &ts);
    const double ms = (ts.tv_sec - ts0.tv_sec) * 1e3 + (ts.tv_nsec - ts0.tv_nsec) * 1e-6;
    if (timeout_ms >= 0 && ms > timeout_ms) { if (status) status->code = OFA_TIMEOUT; return OFA_TIMEOUT; }
    // an abort requested before the launch's own set-up ran may have been cleared by it: keep posting it while the launch lives
    if (c->abort_requested && (++polls % 64) == 0) post_abort(c);
    struct timespec sl = {0, 200000}; nanosleep(&sl, nullptr);
  }
  c->in_flight = false;
  cudaEventElapsedTime(&c->last_ms, c->ev0, c->ev1);
  DevStatus ds; cudaMemcpy(&ds, c->d_status, sizeof ds, cudaMemcpyDeviceToHost);
  if (c->cfg.use_decode) { int scal[8]; cudaMemcpy(scal, c->d_scal, sizeof scal, cudaMemcpyDeviceToHost); c->dec_steps_total = scal[DS_STEP]; }
  if (ds.code != 0 || ds.abort != 0) {
    if (status) { status->code = OFA_DEVICE_ABORT; status->dev_code = ds.code; status->phase = ds.phase; status->task = ds.task; status->block = ds.block; status->aux = ds.aux; }
    std::string nm = (ds.phase >= 0 && ds.phase < (int)c->train_ph.size()) ? c->train_ph[ds.phase].name : "?";
    return fail(c, OFA_DEVICE_ABORT, "device-side bounded wait expired: code " + std::to_string(ds.code) + " phase " + std::to_string(ds.phase) + " (" + nm + ") task " +
                                         std::to_string(ds.task) + " block " + std::to_string(ds.block) + " aux " + std::to_string(ds.aux));
  }
  if (c->C.train_sms > 0) c->steps_total += c->last_nsteps;
  return OFA_OK;
}

extern "C" int ofa_steps_done(const ofa_ctx* c) { return c ? c->steps_total : 0; }
extern "C" float ofa_last_launch_ms(const ofa_ctx* c) { return c ? c->last_ms : 0.f; }
extern "C" int ofa_live(const ofa_ctx* c, ofa_live_t* out) {
  if (!c || !out) return OFA_BAD_ARGUMENT;
  const volatile Live* l = c->h_live;
  out->steps = l->steps; out->loss = l->loss; out->decode_steps = l->dec_steps;
  return OFA_OK;
}
extern "C" int ofa_read_losses(ofa_ctx* c, float* out, size_t n) {
  if (!c || !out || (int)n > c->steps_total) return fail(c, OFA_BAD_ARGUMENT, "more losses requested than steps completed");
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "launch in flight");
  cudaSetDevice(c->device);
  return cudaMemcpy(out, c->d_loss_hist, n * sizeof(float), cudaMemcpyDeviceToHost) == cudaSuccess ? OFA_OK : fail(c, OFA_CUDA_ERROR, "D2H failed");
}
extern "C" int ofa_read_step_times(ofa_ctx* c, unsigned long long* out, size_t n) {
  if (!c || !out || (int)n > c->last_nsteps || !c->d_step_done) return fail(c, OFA_BAD_ARGUMENT, "bad count");
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "launch in flight");
  cudaSetDevice(c->device);
  return cudaMemcpy(out, c->d_step_done, n * sizeof(unsigned long long), cudaMemcpyDeviceToHost) == cudaSuccess ? OFA_OK : fail(c, OFA_CUDA_ERROR, "D2H failed");
}
extern "C" int ofa_num_phases(const ofa_ctx* c) { return c ? (int)c->train_ph.size() : 0; }
extern "C" int ofa_phase_info(const ofa_ctx* c, int phase, char* name, size_t name_cap, int* kind, int* ntasks, unsigned long long* busy_ns) {
  if (!c || phase < 0 || phase >= (int)c->train_ph.size()) return OFA_BAD_ARGUMENT;
  const HostPhase& p = c->train_ph[phase];
  if (name && name_cap) { strncpy(name, p.name.c_str(), name_cap - 1); name[name_cap - 1] = 0; }
  if (kind) *kind = p.d.kind;
  if (ntasks) *ntasks = p.d.ntasks;
  if (busy_ns) { if (c->dry) *busy_ns = 0; else { cudaSetDevice(c->device); cudaMemcpy(busy_ns, c->d_phase_busy + phase, 8, cudaMemcpyDeviceToHost); } }
  return OFA_OK;
}
extern "C" int ofa_phase_window(const ofa_ctx* c, int phase, unsigned long long* first_ns, unsigned long long* last_ns) {
  if (!c || !first_ns || !last_ns || phase < 0 || phase >= (int)c->train_ph.size()) return OFA_BAD_ARGUMENT;
  if (c->dry) { *first_ns = *last_ns = 0; return OFA_OK; }
  cudaSetDevice(c->device);
  const bool ok = cudaMemcpy(first_ns, c->d_phase_first + phase, 8, cudaMemcpyDeviceToHost) == cudaSuccess &&
                  cudaMemcpy(last_ns, c->d_phase_last + phase, 8, cudaMemcpyDeviceToHost) == cudaSuccess;
  return ok ? OFA_OK : OFA_CUDA_ERROR;
}
extern "C" int ofa_phase_wait_ns(const ofa_ctx* c, int phase, unsigned long long* wait_ns) {
  if (!c || !wait_ns || phase < 0 || phase >= (int)c->train_ph.size()) return OFA_BAD_ARGUMENT;
  if (c->dry) { *wait_ns = 0; return OFA_OK; }
  cudaSetDevice(c->device);
  return cudaMemcpy(wait_ns, c->d_phase_busy + c->train_ph.size() + phase, 8, cudaMemcpyDeviceToHost) == cudaSuccess ? OFA_OK : OFA_CUDA_ERROR;
}
extern "C" int ofa_read_block_busy(ofa_ctx* c, unsigned long long* out, size_t n) {
  if (!c || !out || c->dry || n > (size_t)6 * c->nblocks) return fail(c, OFA_BAD_ARGUMENT, "bad request");
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "launch in flight");
  cudaSetDevice(c->device);
  return cudaMemcpy(out, c->d_blk_busy, n * 8, cudaMemcpyDeviceToHost) == cudaSuccess ? OFA_OK : fail(c, OFA_CUDA_ERROR, "D2H failed");
}
extern "C" int ofa_read_decode_trace(ofa_ctx* c, unsigned long long* out, size_t n) {
  if (!c || !out || c->dry || n > 64 || !c->cfg.use_decode) return fail(c, OFA_BAD_ARGUMENT, "bad request");
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "launch in flight");
  cudaSetDevice(c->device);
  return cudaMemcpy(out, c->C.dp.trace, n * 8, cudaMemcpyDeviceToHost) == cudaSuccess ? OFA_OK : fail(c, OFA_CUDA_ERROR, "D2H failed");
}
extern "C" int ofa_read_block_info(ofa_ctx* c, int* out, size_t n) {
  if (!c || !out || c->dry || n > (size_t)c->nblocks) return fail(c, OFA_BAD_ARGUMENT, "bad request");
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "launch in flight");
  cudaSetDevice(c->device);
  return cudaMemcpy(out, c->d_blk_info, n * 4, cudaMemcpyDeviceToHost) == cudaSuccess ? OFA_OK : fail(c, OFA_CUDA_ERROR, "D2H failed");
}
extern "C" int ofa_decode_phase_info(const ofa_ctx* c, int phase, char* name, size_t name_cap, int* ntasks, unsigned long long* busy_ns) {
  if (!c || phase < 0 || phase >= (int)c->dec_ph.size()) return OFA_BAD_ARGUMENT;
  const HostPhase& p = c->dec_ph[phase];
  if (name && name_cap) { strncpy(name, p.name.c_str(), name_cap - 1); name[name_cap - 1] = 0; }
  if (ntasks) *ntasks = p.d.ntasks;
  if (busy_ns) { if (c->dry) *busy_ns = 0; else { cudaSetDevice(c->device); cudaMemcpy(busy_ns, c->d_dec_phase_busy + phase, 8, cudaMemcpyDeviceToHost); } }
  return OFA_OK;
}
extern "C" int ofa_phase_deps(const ofa_ctx* c, int job, int phase, int* dep_phase, int* dep_delta, int cap) {
  if (!c || (job != 0 && job != 1)) return -1;
  const std::vector<HostPhase>& P = job == 0 ? c->train_ph : c->dec_ph;
  if (phase < 0 || phase >= (int)P.size()) return -1;
  const int n = (int)P[phase].deps.size();
  for (int i = 0; i < n && i < cap; i++) { if (dep_phase) dep_phase[i] = P[phase].deps[i].phase; if (dep_delta) dep_delta[i] = P[phase].deps[i].delta; }
  return n;
}
extern "C" int ofa_phase_dep_grain(const ofa_ctx* c, int phase, int* rb_map, int* grain, int cap) {
  if (!c || phase < 0 || phase >= (int)c->train_ph.size()) return -1;
  const HostPhase& p = c->train_ph[phase];
  if (rb_map) *rb_map = p.rb_map;
  const int n = (int)p.deps.size();
  for (int i = 0; i < n && i < cap; i++) if (grain) grain[i] = (i < (int)p.rb_grain.size() && p.rb_grain[i] && p.rb_map && c->train_ph[p.deps[i].phase].rb_map) ? 1 : 0;
  return n;
}
extern "C" int ofa_decode_steps(const ofa_ctx* c) { return c ? c->dec_steps_total : 0; }
extern "C" int ofa_read_decode_tokens(ofa_ctx* c, int* out, size_t cap) {
  if (!c || !out || !c->h_out) return fail(c, OFA_BAD_ARGUMENT, "decode is not enabled");
  const size_t n = std::min(cap, (size_t)c->out_cap);
  const volatile int* src = c->h_out;
  for (size_t i = 0; i < n; i++) out[i] = src[i];
  return (int)n;
}
extern "C" int ofa_read_decode_logits(ofa_ctx* c, float* out, size_t n) {
  if (!c || !out || !c->cfg.use_decode || n > (size_t)c->md.V) return fail(c, OFA_BAD_ARGUMENT, "bad request");
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "launch in flight");
  cudaSetDevice(c->device);
  return cudaMemcpy(out, c->C.dp.st.logits, n * sizeof(float), cudaMemcpyDeviceToHost) == cudaSuccess ? OFA_OK : fail(c, OFA_CUDA_ERROR, "D2H failed");
}
extern "C" int ofa_read_buffer(ofa_ctx* c, const char* name, void* out, size_t bytes) {
  if (!c || !name || !out) return OFA_BAD_ARGUMENT;
  if (c->in_flight) return fail(c, OFA_BAD_ARGUMENT, "launch in flight");
  auto it = c->bufs.find(name);
  if (it == c->bufs.end()) return fail(c, OFA_BAD_ARGUMENT, std::string("no buffer named ") + name);
  if (bytes > it->second.second) return fail(c, OFA_BAD_ARGUMENT, "buffer is smaller than requested");
  cudaSetDevice(c->device);
  return cudaMemcpy(out, it->second.first, bytes, cudaMemcpyDeviceToHost) == cudaSuccess ? OFA_OK : fail(c, OFA_CUDA_ERROR, "D2H failed");
}

// ================================================================================================ C ABI: task level
extern "C" int ofa_dev_alloc(void** p, size_t bytes) {
  if (!p) return OFA_BAD_ARGUMENT;
  if (cudaMalloc(p, bytes ? bytes : 1) != cudaSuccess) { *p = nullptr; return OFA_CUDA_ERROR; }
  cudaMemset(*p, 0, bytes);
  return OFA_OK;
}
extern "C" int ofa_dev_free(void* p) { return cudaFree(p) == cudaSuccess ? OFA_OK : OFA_CUDA_ERROR; }
extern "C" int ofa_h2d(void* dst, const void* src, size_t bytes) { return cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice) == cudaSuccess ? OFA_OK : OFA_CUDA_ERROR; }
extern "C" int ofa_d2h(void* dst, const void* src, size_t bytes) { return cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost) == cudaSuccess ? OFA_OK : OFA_CUDA_ERROR; }

extern "C" int ofa_run_phases(int dtype, const ofa_dims* dims, const ofa_phase* phases, int nph, int repeats, const float* adam,
                              float* ms, ofa_status_t* status) {
  if (status) memset(status, 0, sizeof *status);
  if (!dims || !phases || nph <= 0 || repeats <= 0 || (dtype != OFA_DTYPE_BF16 && dtype != OFA_DTYPE_F32)) return fail(nullptr, OFA_BAD_ARGUMENT, "bad argument");
  const bool bf = dtype == OFA_DTYPE_BF16;
  ModelDims m{};
  m.V = dims->vocab; m.D = dims->d_model; m.L = dims->n_layer; m.H = dims->n_head; m.T = dims->ctx_len; m.B = dims->batch; m.N = m.B * m.T; m.FF = 4 * m.D;
  m.DH = m.H > 0 ? m.D / m.H : 0; m.valid_vocab = m.V;
  if (m.V <= 0 || m.H <= 0 || m.T <= 0 || m.B <= 0) return fail(nullptr, OFA_BAD_CONFIG, "non-positive dimension");
  if (bf ? (m.D != 768 || m.DH != 64) : (m.D != 64 || m.DH != 16)) return fail(nullptr, OFA_BAD_CONFIG, "unsupported width / head dim for this dtype");
  const int smem = smem_for(bf, m.T, m.N);
  {  // sizes that do not fit a block are refused before anything touches the device
    bool emb = false;
    for (int i = 0; i < nph; i++) emb = emb || phases[i].kind == TK_EMB_WTE;
    const std::string e = smem_fit_error(bf, m.T, m.N, emb, false, smem);
    if (!e.empty()) return fail(nullptr, OFA_BAD_CONFIG, e);
  }
  int dev = 0; cudaDeviceProp prop;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return fail(nullptr, OFA_CUDA_ERROR, "no CUDA device");
  if (prop.major != 10) return fail(nullptr, OFA_CUDA_ERROR, "sm_100a code only");
  const int nblocks = 2 * prop.multiProcessorCount;
  Arena ar; DevJob dj; std::string err;
  std::vector<HostPhase> P(nph);
  for (int i = 0; i < nph; i++) {
    const ofa_phase& s = phases[i];
    HostPhase& hp = P[i]; hp.name = "phase" + std::to_string(i);
    PhaseDesc& d = hp.d; memset(&d, 0, sizeof d);
    d.kind = s.kind; d.layout = s.layout; d.epi = s.epi; d.i0 = s.i0; d.i1 = s.i1; d.i2 = s.i2; d.n = s.n;
    for (int k = 0; k < 10; k++) d.p[k] = s.p[k];
    const int BH = m.B * m.H, rows16 = (m.N + 15) / 16;
    switch (s.kind) {
      case TK_GEMM:
        d.g.A = s.p[0]; d.g.B = s.p[1]; d.g.C = s.p[2]; d.g.aux = s.p[3]; d.g.M = s.M; d.g.N = s.N; d.g.K = s.K; d.g.lda = s.lda; d.g.ldb = s.ldb; d.g.ldc = s.ldc; d.g.ldaux = s.ldaux;
        d.g.accumulate = s.accumulate;
        if (s.epi == GE_LSE) {  // p[4] = softmax partials [M, N / 128] float2
          if (!bf || !s.p[4] || s.layout != GL_NT) { ar.free_all(); return fail(nullptr, OFA_BAD_ARGUMENT, "softmax-partial epilogue: bf16, NT layout, p[4] = output [M, N/128] float2"); }
          d.g.dr = reinterpret_cast<float*>(s.p[4]);
        }
        if (s.epi == GE_DR) {   // p[4] = row-term output [B, H, T]; needs the tensor-core path, heads of 64 columns and whole rows of heads in C
          if (!bf || !s.p[4] || s.layout != GL_NT || s.N != m.D || s.M != m.N) { ar.free_all(); return fail(nullptr, OFA_BAD_ARGUMENT, "row-term epilogue: bf16, NT layout, C = [tokens, d_model], p[4] = output"); }
          d.g.dr = reinterpret_cast<float*>(s.p[4]); d.g.dr_T = m.T; d.g.dr_H = m.H;
        }
        if (bf) { if (!prepare_gemm_bf16(d, ar, s.nsub, nblocks, err)) { ar.free_all(); return fail(nullptr, OFA_BAD_ARGUMENT, err); } }
        else prepare_gemm_f32(d);
        break;
      case TK_EMBED: case TK_LN_FWD: case TK_LN_BWD: d.ntasks = rows16; break;
      case TK_LN_DG: d.ntasks = (m.D + NTHR - 1) / NTHR; break;
      case TK_ATT_FWD: d.ntasks = bf ? BH * (m.T / attn::QTILE) : BH;
        if (bf) { d.p[6] = const_cast<void*>(make_attn_maps(ar, s.p[0], nullptr, m.N, m.D, err)); if (!d.p[6]) { ar.free_all(); return fail(nullptr, OFA_CUDA_ERROR, err); } }
        break;
      case TK_ATT_PREP: d.ntasks = bf ? BH * (m.T / attn::QTILE) : 1; break;
      case TK_ATT_BWD: d.ntasks = bf ? 2 * BH * (m.T / attn::QTILE) : BH;
        if (bf) { d.p[6] = const_cast<void*>(make_attn_maps(ar, s.p[0], s.p[1], m.N, m.D, err)); if (!d.p[6]) { ar.free_all(); return fail(nullptr, OFA_CUDA_ERROR, err); } }
        break;
      case TK_CE: d.ntasks = (m.N + ew::CE_ROWS - 1) / ew::CE_ROWS;
        if (s.p[3]) { if (!bf || m.V % 128) { ar.free_all(); return fail(nullptr, OFA_BAD_ARGUMENT, "cross-entropy with softmax partials: bf16, vocab a multiple of 128"); } d.i2 = m.V / 128; }
        d.i0 = (int)(std::min<size_t>((size_t)((bf ? gemm_tc::BAR_OFFSET : smem - CTRL_BYTES) - 64), (size_t)m.V * (bf ? 2 : 4)) / 16 * 16); break;
      case TK_CE_MEAN: d.ntasks = 1; break;
      case TK_BARRIER: d.ntasks = s.n > 0 ? (int)std::min<size_t>(s.n, 1u << 24) : 1; break;     // n empty tasks: what a task costs the scheduler alone
      case TK_EMB_WTE: d.ntasks = (m.V + ew::EMB_VCHUNK - 1) / ew::EMB_VCHUNK; break;
      case TK_EMB_WPE: d.ntasks = (m.T + ew::WPE_ROWS - 1) / ew::WPE_ROWS; break;
      case TK_ADAMW: d.ntasks = (int)((s.n + ew::OPT_CHUNK - 1) / ew::OPT_CHUNK); if (s.n == 0 || s.n % 4) { ar.free_all(); return fail(nullptr, OFA_BAD_ARGUMENT, "AdamW n must be a positive multiple of 4"); } break;
      default: ar.free_all(); return fail(nullptr, OFA_BAD_ARGUMENT, "task kind not available at task level");
    }
    if (bf && (s.kind == TK_ATT_FWD || s.kind == TK_ATT_BWD || s.kind == TK_ATT_PREP) && m.T % attn::QTILE) { ar.free_all(); return fail(nullptr, OFA_BAD_ARGUMENT, "ctx_len must be a multiple of 128"); }
    if (i > 0) hp.deps.push_back(Dep{i - 1, 0});
  }
  P[0].deps.push_back(Dep{nph - 1, -1});
  if (!upload_job(P, nph - 1, repeats, dj, err)) { ar.free_all(); return fail(nullptr, OFA_BAD_ARGUMENT, err); }
  static thread_local Ctx C;      // 31 KB: not on the stack
  memset(&C, 0, sizeof C);
  C.train = dj.j; C.md = m;
  fill_param_records(C, &dj, nullptr);
  if (adam) { C.hp.lr_max = adam[0]; C.hp.lr_min = adam[0]; C.hp.beta1 = adam[1]; C.hp.beta2 = adam[2]; C.hp.eps = adam[3]; C.hp.wd = adam[4]; C.hp.grad_scale = adam[5]; C.hp.constant_lr = 1; }
  C.train_sms = prop.multiProcessorCount; C.use_train = 1;
  C.status = ar.alloc<DevStatus>(1); C.finished = ar.alloc<int>(1); C.t_end = ar.alloc<unsigned long long>(1);
  C.step_done = ar.alloc<unsigned long long>(repeats); C.loss_hist = ar.alloc<float>(repeats);
  C.tok_in = nullptr; C.tok_tgt = nullptr;
  C.dep_timeout_ns = 20000000000ull;
  C.smem_bytes = smem;
  C.prof_step = -1;
  if (!ar.ok) { ar.free_all(); dj.free_all(); return fail(nullptr, OFA_CUDA_ERROR, "out of device memory"); }
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  cudaEventRecord(e0, 0);
  cudaError_t e = bf ? launch_kernel<bf16, 768, 64>(C, nblocks, smem, 0) : launch_kernel<float, 64, 16>(C, nblocks, smem, 0);
  cudaEventRecord(e1, 0);
  int rc = OFA_OK;
  if (e != cudaSuccess) { rc = fail(nullptr, OFA_CUDA_ERROR, std::string("launch failed: ") + cudaGetErrorString(e)); }
  else if ((e = cudaEventSynchronize(e1)) != cudaSuccess) { rc = fail(nullptr, OFA_CUDA_ERROR, std::string("kernel failed: ") + cudaGetErrorString(e)); }
  else {
    float t = 0.f; cudaEventElapsedTime(&t, e0, e1); if (ms) *ms = t;
    DevStatus ds; cudaMemcpy(&ds, C.status, sizeof ds, cudaMemcpyDeviceToHost);
    if (ds.code || ds.abort) {
      if (status) { status->code = OFA_DEVICE_ABORT; status->dev_code = ds.code; status->phase = ds.phase; status->task = ds.task; status->block = ds.block; status->aux = ds.aux; }
      rc = fail(nullptr, OFA_DEVICE_ABORT, "device-side bounded wait expired: code " + std::to_string(ds.code) + " phase " + std::to_string(ds.phase) + " task " + std::to_string(ds.task) + " aux " + std::to_string(ds.aux));
    }
  }
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  ar.free_all(); dj.free_all();
  return rc;
}

// Test hook: seed != 0 makes every phase uploaded afterwards (ofa_launch, ofa_run_phases) hand its tasks out in a permuted order;
// 0 restores the natural order. Results must be bit-identical either way (llm/gemm/test_gemm.cu:20-49 checks the same property).
extern "C" void ofa_debug_set_task_shuffle(unsigned seed) { g_task_shuffle_seed = seed; }

// ================================================================================================ C ABI: data-parallel hooks
extern "C" int ofa_num_buckets(const ofa_ctx* c) { return c ? (int)c->buckets.size() : 0; }
extern "C" int ofa_bucket_span(const ofa_ctx* c, int b, size_t* offset, size_t* count) {
  if (!c || b < 0 || b >= (int)c->buckets.size()) return OFA_BAD_ARGUMENT;
  if (offset) *offset = c->buckets[b].off;
  if (count) *count = c->buckets[b].n;
  return OFA_OK;
}
extern "C" void* ofa_grad_buffer(const ofa_ctx* c) { return c ? (c->cfg.grad_bf16 ? (void*)c->Gbf : (void*)c->G32) : nullptr; }
extern "C" int* ofa_ext_ready_flags(const ofa_ctx* c) { return c ? c->d_ext_ready : nullptr; }
extern "C" int* ofa_ext_done_flags(const ofa_ctx* c) { return c ? c->d_ext_done : nullptr; }

#include "dp_nccl.inc"
