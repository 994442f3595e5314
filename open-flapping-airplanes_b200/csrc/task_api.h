// The task API of the megakernel: what a phase is, how a job (a cyclic table of phases with dependency counters) is laid
// out in device memory, and the context the one persistent launch receives. Shared by host (graph builder) and device.
//
// It keeps the model of the reference program's `PhaseDesc / Job / Ctx` (llm/b200/megakernel/ofa.cu:87-117): a phase is
// `ntasks` independent block-sized tasks of one kind; a job is the list of phases of one step, executed for `nsteps`
// steps; a global ticket counter hands out (step, phase, task) in topological order; `done[phase]` counts finished tasks
// monotonically over all steps, and a dependency (phase p, step delta d) of a task in step s is satisfied when
// done[p] >= ntasks[p] * (s + 1 + d).
#pragma once
#include <stdint.h>
#include <stddef.h>

namespace ofa {

enum TaskKind : int {
  TK_DATA = 0,     // copy this step's token windows into tok_in / tok_tgt
  TK_EMBED,        // x0 = wte[tok] + wpe[pos]
  TK_LN_FWD,
  TK_GEMM,         // tensor-core (bf16) or SIMT (fp32) GEMM tile strip, see GemmArgs
  TK_ATT_FWD,
  TK_ATT_PREP,     // D = rowsum(dO * O)
  TK_ATT_BWD,      // first half of the tasks: dK/dV, second half: dQ
  TK_CE,           // in-place logits -> dlogits, per-row loss
  TK_CE_MEAN,
  TK_LN_BWD,
  TK_LN_DG,        // reduce per-task dgamma partials
  TK_EMB_WTE,
  TK_EMB_WPE,
  TK_ADAMW,
  TK_BARRIER,      // 1 task, does nothing: its completion marks the end of a step
  TK_DEC_QKV,      // decode job: i0 = layer
  TK_DEC_ATTWO,
  TK_DEC_UPDN,
  TK_DEC_HEAD,
  TK_DEC_SAMPLE,
  TK_EXT_WAIT,     // 1 task: wait (bounded) until an external 32-bit flag >= step_base+step+1 (gradient all-reduce finished)
  TK_SUMCAST,      // out[i] = act(sum of i0 fp32 partial buffers p[1..]) over n elements (split-K reduce)
  TK_EXT_SIGNAL,   // 1 task: store step_base+step+1 to an external 32-bit flag (gradient bucket ready)
  TK_COUNT
};

enum GemmLayout : int { GL_NN = 0, GL_NT = 1, GL_TN = 2 };
// NN: C[M,N] = A[M,K] . B[K,N]      NT: C = A[M,K] . B[N,K]^T      TN: C = A[K,M]^T . B[K,N]      (all row-major)
enum GemmEpi : int {
  GE_STORE = 0,   // C = act(acc)                       (activation storage type)
  GE_RES,         // C = act(acc + aux)                 (aux may alias C)
  GE_GELU,        // aux = act(acc); C = act(gelu(aux)) (pre-activation saved for backward)
  GE_DGELU,       // C = act(acc * gelu'(aux))
  GE_F32,         // C(fp32) = acc, or C += acc when `accumulate`
  GE_DR,          // C = act(acc); dr[b, h, t] = sum over head h's 64 columns of float(C) * aux   (attention backward's row term,
                  // with C = dO and aux = O; tensor-core path only)
  GE_LSE,         // C = act(acc); lse_part[row, tile_n] = {m, s}: m = max over the tile's 128 stored (rounded) values of x * log2(e),
                  // s = sum of 2^(x * log2(e) - m)   (softmax partials of the LM head: cross-entropy then needs one pass over the
                  // logits instead of two; tensor-core path only)
};

struct GemmArgs {
  const void* A; const void* B; void* C; void* aux;
  int M, N, K;
  int lda, ldb, ldc, ldaux;   // leading dimensions in elements
  int accumulate;             // GE_F32 only
  int nsub;                   // consecutive N tiles handled by one task (tensor-core path)
  int bn;                     // tile width of the tensor-core path: 256 when N is a multiple of 256, else 128
  const void* tmA;            // device pointers to the two TMA descriptors (tensor-core path), 64-byte aligned
  const void* tmB;
  float* dr; int dr_T, dr_H;  // GE_DR: output [B, H, T] and its dimensions (row = b * T + t, head = column / 64). GE_LSE: dr = output [M, N / 128] float2
};

struct alignas(16) PhaseDesc {
  int kind, ntasks, layout, epi;
  int tiles_m, i0, i1, i2;
  GemmArgs g;
  void* p[10];
  size_t n;
  float f0, f1;
};

struct Dep { int phase; int delta; };   // need done[phase] >= ntasks[phase] * (step + 1 + delta)

// Everything the scheduler thread needs to place a ticket in a phase and to check that phase's dependencies, in one 64-byte
// line: one memory round trip per phase change instead of a chain of dependent table look-ups.
//
// Dependencies come in two grains. A phase-level dependency (the reference's only kind, ofa.cu:245-255) waits until EVERY task of
// the producer phase has finished. A row-block dependency waits only for the producer tasks that write the 128-token row blocks
// the waiting task reads: the producer counts its completions per row block as well (Job::done_rb), and the consumer derives the
// row blocks it needs from its own task index (rb_map). Consecutive phases of the layer chain (LayerNorm -> GEMM -> attention ->
// GEMM ...) then overlap instead of meeting at a barrier after every phase.
enum RbKind : int {
  RB_NONE = 0,
  RB_MOD,        // task -> row block task % a            (GEMM strips: a = tiles along M, consecutive tasks walk down M)
  RB_DIV,        // task -> row block task / a            (row-wise tasks: a = tasks per 128 rows)
  RB_ATT_FWD,    // attention forward task (b, h, query tile): writes its query tile's row block, reads row blocks 0..tile of sequence b
  RB_ATT_BWD,    // attention backward: dK/dV task (key tile) reads row blocks tile..last of its sequence; dQ task its own row block
};
struct alignas(16) SchedRec {
  int lo, hi;               // tickets [lo, hi) of a step belong to this phase
  int ndeps;                // 0..4 dependencies held in dep[]; -1: more than four, use Job::deps (phase-level only)
  int perm_mul;             // 0 (production), or a multiplier coprime with the task count: ticket i of the phase runs task (i * perm_mul + perm_mul / 2) % ntasks (test hook: results must not depend on the order)
  int rb_off;               // where this phase counts completions per row block in Job::done_rb, -1: it does not
  int rb_map;               // RbKind | a << 8
  int dep[8];               // per dependency: {phase | (step delta == -1) << 16 | row-block grain << 17,  completions needed per step: tasks of the phase, or tasks per row block}
  int pad[2];
};
constexpr int DEP_PREV = 1 << 16, DEP_RB = 1 << 17;
constexpr int CTRL_BYTES = 1024;   // control area at the end of every block's dynamic shared memory
// The scheduling records of both jobs travel with the launch as part of the kernel parameter (constant bank): a block that
// claims a ticket finds the phase and its dependencies without a single round trip to global memory. Jobs with more phases than
// fit (the parameter is limited to 32,764 bytes) fall back to the records in global memory.
constexpr int PARAM_TRAIN_PH = 400, PARAM_DEC_PH = 64;

struct Job {
  int nph, tasks_per_step, nsteps, last_phase;
  const PhaseDesc* ph;      // [nph]
  const int* prefix;        // [nph+1] exclusive prefix sum of ntasks
  const int* ntasks;        // [nph]
  const int* dep_off;       // [nph]
  const int* dep_cnt;       // [nph]
  const Dep* deps;
  const SchedRec* rec;      // [nph]
  int* done;                // [nph] monotonically increasing over steps
  int* done_rb;             // completions per (phase that publishes them, row block of 128 tokens), monotonically increasing; see SchedRec
  unsigned* ticket;         // next (step * tasks_per_step + task) to hand out
};

struct ModelDims { int V, D, L, H, T, B, N, FF, DH, valid_vocab; };

struct AdamConst { float lr_max, lr_min, beta1, beta2, eps, wd; int warmup, sched_steps, constant_lr; float grad_scale; };

// pinned, host-mapped words the device updates while running; any host thread may read them
struct Live { unsigned steps; float loss; unsigned dec_steps; unsigned pad; };

constexpr int OUT_RESTART = 1 << 24;       // out_tokens marker: a new answer starts (prompt about to be fed)
constexpr int OUT_FORCED = OUT_RESTART + 1; // out_tokens marker: a prompt token was fed (no sample kept)

struct DecodeState {       // device memory; fixed-point residual makes the task order irrelevant to the result
  unsigned long long* xw;  // [D] residual, int64 in 2^-30 units (master copy)
  unsigned long long* xr;  // [D] copy read by the MLP task
  void* q;                 // [D] activation type
  float* cand_v;           // [2][nchunk]
  int* cand_i;             // [2][nchunk]
  int* scal;               // token, pos, step, ctx_full, astep
  void* kv;                // [L][2][H][T][DH] activation type
  float* logits;           // [V]
  int* out_tokens;         // pinned ring [out_cap]
  int out_cap;
};
enum { DS_TOKEN = 0, DS_POS = 1, DS_STEP = 2, DS_CTXFULL = 3, DS_ASTEP = 4,
       DS_POSKEY = 5,   // (context epoch << 16) | pos in ONE word: a prefetch made ahead of time can tell whether the rows it copied belong to the context the task finally runs in
       DS_EPOCH = 6 };

struct DecodeParams {
  // weights: pointers into the SAME working-copy buffer the trainer updates
  const void *wte, *wpe, *head, *gf;
  const void* const* wqkv; const void* const* wo; const void* const* wup; const void* const* wdn;
  const void* const* g1; const void* const* g2;   // device arrays [L]
  const void *tm_qkv, *tm_up, *tm_wo;             // device arrays [L] of 128-byte TMA descriptors (unswizzled 2-D views of Wqkv, Wup, Wo) for the weight prefetch
  DecodeState st;
  float temperature;       // <= 0: greedy
  unsigned long long seed;
  const int* forced; int nforced;
  int auto_reset, answer_len;
  int max_steps;           // stop decoding after this many tokens (0 = until training finishes)
  unsigned long long* trace;   // optional: 64 %globaltimer stamps of stage boundaries inside serving task 0 of layer 0
};

struct DevStatus;

struct Ctx {
  Job train, dec;
  ModelDims md;
  AdamConst hp;
  const uint32_t* data; unsigned long long ntok; const uint32_t* starts; int nstarts; unsigned long long seed;
  int* tok_in; int* tok_tgt;
  int step_base;            // steps completed by earlier launches: added to the step index for data windows, LR and AdamW
  unsigned long long *phase_busy, *phase_first, *phase_last; int prof_step;
  unsigned long long* blk_wait;         // per block: time its thread 0 spent waiting for training dependencies (ns)
  unsigned long long* dec_phase_busy;   // per serving phase: summed task time (ns)
  unsigned long long* step_done; float* loss_hist; unsigned long long* blk_busy; int* finished; unsigned long long* t_end;
  int infer_sms, reserved_sms, train_sms, use_decode, use_train;
  const int* smid_rank;     // %smid -> dense SM rank (nullptr = identity)
  DecodeParams dp;
  Live* live;
  DevStatus* status;
  unsigned long long dep_timeout_ns;
  int* blk_info;            // per block: %smid | role << 16 (1 serve, 2 reserved-idle, 3 train, 4 idle)
  int* arrived;             // blocks of this launch that have started (idle partitions leave only when all have)
  int smem_bytes;           // dynamic shared memory per block; its last 1,024 bytes are the control area (barriers, hand-off words, descriptor slots)
  int sched_flags;                          // bit 1: keep the per-phase / per-block time tables
  int train_rec_n, dec_rec_n;               // phases whose records are held below (0: use Job::rec in global memory)
  SchedRec train_rec[PARAM_TRAIN_PH];
  SchedRec dec_rec[PARAM_DEC_PH];
};
static_assert(sizeof(Ctx) <= 32764, "kernel parameter too large");

}  // namespace ofa
