/* C ABI of libofa_b200.so: a B200-native persistent megakernel that trains a GPT and serves it from the live weights.
 *
 * The reference program (Bobliuuu/open-flapping-airplanes, llm/b200/megakernel/ofa.cu) has no library boundary: its
 * main() builds the phase tables, uploads them and performs the one launch. This header exports exactly what that
 * main() does, split into calls a host program (C++, or Python through ctypes) can drive. Every entry point cites the
 * part of the reference it replaces. Plain pointers and sizes only; the caller owns host buffers, the library owns
 * device memory. No call blocks forever and no call exits the process: errors come back as ofa_status codes and
 * ofa_last_error() gives the text.
 *
 * Two levels:
 *   model level  - ofa_create / ofa_load_weights / ofa_set_tokens / ofa_launch / ofa_wait / ofa_read_*  (ofa.cu:394-766)
 *   task level   - ofa_run_phases: run an explicit list of phase descriptors through the same persistent scheduler; this
 *                  is the reference's task API (PhaseDesc/Job, ofa.cu:87-117) and what its per-library tests drive
 *                  (llm/gemm/test_gemm.cu:20-49, llm/attention/test_attention.cu:45-77, llm/elementwise/test_elementwise.cu:19-47).
 */
#ifndef OFA_B200_H
#define OFA_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ofa_ctx ofa_ctx;

typedef enum {
  OFA_OK = 0,
  OFA_TIMEOUT = 1,        /* ofa_wait: the launch is still running after timeout_ms                       */
  OFA_DEVICE_ABORT = 2,   /* a bounded device-side wait expired; see ofa_status_t.{code,phase,task,block}  */
  OFA_CUDA_ERROR = 3,
  OFA_BAD_CONFIG = 4,
  OFA_BAD_ARGUMENT = 5,
  OFA_NOT_LAUNCHED = 6
} ofa_code;

typedef struct {
  int code;               /* ofa_code */
  int dev_code;           /* device status: 1 dependency timeout, 2/3/4 mbarrier timeouts, 5 smem misaligned, 6 external flag timeout, 7 bad descriptor */
  int phase, task, block, aux;
} ofa_status_t;

enum { OFA_DTYPE_BF16 = 0, OFA_DTYPE_F32 = 1 };
enum { OFA_MODE_TRAIN = 0, OFA_MODE_FORWARD = 1, OFA_MODE_NO_OPT = 2, OFA_MODE_DECODE_ONLY = 3 };

/* Replaces the compile-time constants and argv/env flags of the reference (ofa.cu:61-84, 395-430, 696). */
typedef struct {
  int vocab, d_model, n_layer, n_head, ctx_len, batch;   /* ffn = 4*d_model, head_dim = d_model/n_head           */
  int valid_vocab;          /* ids >= valid_vocab are never sampled (ofa.cu:71 VALID)                             */
  int tied_head;            /* 1: LM head = wte (reference), 0: separate lm_head[V,D] after wpe in the flat layout */
  int dtype;                /* OFA_DTYPE_BF16: d_model 768 / head_dim 64, tensor cores; OFA_DTYPE_F32: d_model 64 / head_dim 16 */
  int mode;                 /* OFA_MODE_*: full training step; forward through logits only; forward+backward without AdamW (ofa.cu --no-opt); or no training job at all (serving only: ofa_launch counts decode tokens) */
  int sched_steps, warmup, constant_lr;
  float lr_max, lr_min, beta1, beta2, eps, weight_decay;
  unsigned long long data_seed;   /* window starts when no starts table is set (ofa.cu:160) */
  int infer_sms, reserved_sms, train_sms;   /* SM split (ofa.cu:384-391); train_sms <= 0: all remaining SMs       */
  int use_decode;           /* run the serving job concurrently                                                   */
  int n_prompt; int prompt[32]; int answer_len; float temperature; unsigned long long decode_seed;
  int decode_out_cap;       /* size of the pinned token ring                                                      */
  int dp_world;             /* gradient scale 1/dp_world is folded into AdamW                                      */
  int grad_bf16;            /* weight gradients are written as bf16 (the all-reduce bucket format)                */
  int ext_sync;             /* 1: gradients are cut into buckets; the graph raises a "ready" flag per bucket and holds the bucket's AdamW until the matching "done" flag is raised from outside (the all-reduce) */
  int bucket_bytes;         /* target bucket size for ext_sync (0 = 25 MiB)                                       */
  int attn_legacy;          /* must be 0 (the field once selected mma.sync attention tasks kept for comparison; they are gone, the tensor-core tasks are checked against the oracle directly) */
  int adam_interleave;      /* experimental, default 0: 1 = each layer's AdamW phase inside the backward pass; n >= 2 = AdamW trickles through the backward pass, up to n tasks after every backward phase */
  int head_dx_splitk;       /* 1: compute lm_head dX as K-split partial products + reduce (experimental, default 0)     */
  int gemm_nsub;            /* consecutive N tiles per GEMM task: n = strips of n 128-wide tiles; 0 = chosen per phase by waves over the blocks that train; 2000 + n = 256-wide tiles where N allows; 4000 + n = the same with a phase's tasks ordered along N first (also accepted as ofa_phase.nsub) */
  double timeout_s;         /* device-side bound for a wait on an external flag (0 = default 20 s); waits for dependencies inside the graph give up after 1.5 x this */
  int device;               /* CUDA device ordinal; < 0 = planning context: layout, buckets and phase graphs are built and can be queried, nothing touches a device and nothing can be launched */
  int sched_profile;        /* 1 (preset default): the kernel keeps the per-phase and per-block time tables that ofa_phase_info / ofa_phase_wait_ns / ofa_phase_window / ofa_read_block_busy / ofa_read_decode_trace report (the reference's report section, ofa.cu:722-746); 0: it does not (they read zero) and every task saves several timer reads and atomics. Step times, losses and live words are kept either way */
} ofa_config;

/* preset: "tiny" (the char-level fp32 model: vocab 65, d_model 64, 2 layers, 4 heads, context 64, batch 16) or "gpt_s" (the 162M bf16 model: vocab 50304 untied, d_model 768, 12 layers, 12 heads, context 1024, batch 4). */
int ofa_default_config(ofa_config* cfg, const char* preset);

/* lifecycle: replaces the body of main() up to the launch (ofa.cu:415-707). One ctx per device. */
int ofa_create(const ofa_config* cfg, ofa_ctx** out);
void ofa_destroy(ofa_ctx* ctx);
const char* ofa_last_error(const ofa_ctx* ctx);   /* ctx may be NULL: error of the last failed ofa_create on this thread */

/* flat parameter layout (ofa.cu:338-350 `struct Layout`): wte, wpe, [lm_head], per layer {g1, Wqkv, Wo, g2, Wup, Wdn}, gf */
size_t ofa_num_params(const ofa_ctx* ctx);
/* name: "wte","wpe","lm_head","gf","L<l>.g1|Wqkv|Wo|g2|Wup|Wdn". Returns 0 and fills offset/count (elements), or OFA_BAD_ARGUMENT. */
int ofa_param_span(const ofa_ctx* ctx, const char* name, size_t* offset, size_t* count);

/* weights in/out: replaces --init / --dump-w / --dump-grads (ofa.cu:491, 762-763). fp32, flat layout order. */
int ofa_load_weights(ofa_ctx* ctx, const float* flat, size_t n);
int ofa_read_weights(ofa_ctx* ctx, float* out, size_t n);
int ofa_read_grads(ofa_ctx* ctx, float* out, size_t n);     /* converted to fp32 when grad_bf16 */
int ofa_read_adam_m(ofa_ctx* ctx, float* out, size_t n);
int ofa_read_adam_v(ofa_ctx* ctx, float* out, size_t n);
int ofa_load_adam_state(ofa_ctx* ctx, const float* m, const float* v, size_t n, int step_base);   /* resume */

/* tokens: replaces --data / --starts (ofa.cu:513-528). starts is [nsteps][batch] window offsets, or NULL for hashed starts.
 * ofa_set_tokens drops a starts table set earlier (it was checked against the old stream): set tokens first, then starts. */
int ofa_set_tokens(ofa_ctx* ctx, const uint32_t* tokens, size_t n);
int ofa_set_starts(ofa_ctx* ctx, const uint32_t* starts, size_t nsteps);

/* run: replaces the launch + event polling loop (ofa.cu:710-716). ofa_launch is asynchronous and runs `nsteps` more
 * training steps (or, without a training job, `nsteps` decode tokens) in ONE persistent launch; ofa_wait returns
 * OFA_TIMEOUT if it is still running after timeout_ms, OFA_DEVICE_ABORT if a bounded device wait expired. */
int ofa_launch(ofa_ctx* ctx, int nsteps);
int ofa_wait(ofa_ctx* ctx, int timeout_ms, ofa_status_t* status);
/* asks a running launch to stop: the device's bounded waits see the request and the kernel returns (ofa_wait then reports OFA_DEVICE_ABORT). ofa_destroy does this itself, waits a few seconds and never blocks for good. */
int ofa_abort(ofa_ctx* ctx);
int ofa_steps_done(const ofa_ctx* ctx);                       /* total training steps completed by finished launches */
float ofa_last_launch_ms(const ofa_ctx* ctx);                 /* CUDA-event time of the last finished launch */

/* live telemetry: the pinned words the device updates while running (doom_job.cuh:29 `Live`, ofa.cu:193,307). */
typedef struct { unsigned steps; float loss; unsigned decode_steps; } ofa_live_t;
int ofa_live(const ofa_ctx* ctx, ofa_live_t* out);

/* results: replaces the report section (ofa.cu:722-756). */
int ofa_read_losses(ofa_ctx* ctx, float* out, size_t n);                  /* loss_hist[0..n) since creation           */
int ofa_read_step_times(ofa_ctx* ctx, unsigned long long* out, size_t n); /* %globaltimer ns at the end of each step of the last launch */
int ofa_num_phases(const ofa_ctx* ctx);
int ofa_phase_info(const ofa_ctx* ctx, int phase, char* name, size_t name_cap, int* kind, int* ntasks, unsigned long long* busy_ns);
/* nanoseconds the training blocks spent waiting for the dependencies of tasks of this phase during the last launch (summed over blocks): shows which phase boundaries the step loses time at; no counterpart in the reference's report */
int ofa_phase_wait_ns(const ofa_ctx* ctx, int phase, unsigned long long* wait_ns);
/* %globaltimer ns at which the first task of the phase started and the last one ended, in the LAST step of the last launch (the "phase wall-clock at step" table of the report, ofa.cu:735-743); first = all ones when the phase had no task in that step */
int ofa_phase_window(const ofa_ctx* ctx, int phase, unsigned long long* first_ns, unsigned long long* last_ns);
/* busy nanoseconds of every block in the last launch: out[2*block + job] (job 0 training, 1 serving) for the first 2*grid entries (ofa.cu:313 blk_busy), then four rows of grid entries each: time the block's scheduler thread spent waiting for training dependencies, claiming tickets, handing the task to the block, and signalling completion; n <= 6 * grid size */
int ofa_read_block_busy(ofa_ctx* ctx, unsigned long long* out, size_t n);
/* in-kernel trace of the serving job (the reference's DTRACE, decode_wide.cuh:11-16): %globaltimer stamps of the stage boundaries inside task 0 of layer 0 (slots 0-4 QKV, 8-12 UP+DOWN, 16-19 scheduler-side start/end of those tasks), last token of the last launch */
int ofa_read_decode_trace(ofa_ctx* ctx, unsigned long long* out, size_t n);
/* where each block of the last launch ran and as what: out[block] = %smid | role << 16, role 1 serving, 2 reserved (idle), 3 training, 4 idle (ofa_kernel's role dispatch, ofa.cu:316-326) */
int ofa_read_block_info(ofa_ctx* ctx, int* out, size_t n);
/* serving-graph counterpart of ofa_phase_info: summed task time of a decode phase during the last launch; returns OFA_BAD_ARGUMENT past the last phase */
int ofa_decode_phase_info(const ofa_ctx* ctx, int phase, char* name, size_t name_cap, int* ntasks, unsigned long long* busy_ns);
/* dependencies of a phase: job 0 = training graph, 1 = serving graph; returns their number and fills up to cap (phase, step-delta) pairs (Job::deps, ofa.cu:103-105) */
int ofa_phase_deps(const ofa_ctx* ctx, int job, int phase, int* dep_phase, int* dep_delta, int cap);
/* grain of the dependencies of a training phase, in the order ofa_phase_deps lists them: grain[i] = 1 when the phase's tasks wait for that producer per 128-token row block (only for the producer tasks that write the rows they read) instead of for the whole producer phase, which is the reference's only grain (ofa.cu:245-255); rb_map = how the phase's own tasks map to row blocks (0: they do not). Returns the number of dependencies. */
int ofa_phase_dep_grain(const ofa_ctx* ctx, int phase, int* rb_map, int* grain, int cap);
int ofa_decode_steps(const ofa_ctx* ctx);                                  /* tokens processed by the serving job      */
int ofa_read_decode_tokens(ofa_ctx* ctx, int* out, size_t cap);            /* the pinned ring: sampled ids, OFA_OUT_* markers, -1 = unused */
int ofa_read_decode_logits(ofa_ctx* ctx, float* out, size_t n);            /* fp32 logits of the last decoded token    */
#define OFA_OUT_RESTART (1 << 24)
#define OFA_OUT_FORCED ((1 << 24) + 1)
/* named activation / gradient buffers for parity checks: "logits","lnf","x<l>","qkv<l>","att<l>","dx<l>", ... */
int ofa_read_buffer(ofa_ctx* ctx, const char* name, void* out, size_t bytes);

/* data-parallel hooks (no counterpart in the single-GPU reference): the gradient buffer (bf16 when grad_bf16, else fp32),
 * its buckets, and the two device flag arrays (int32 per bucket). The communication side waits until ready[b] >= s+1,
 * all-reduces bucket b in place, then stores s+1 to done[b], where s counts steps since ofa_create (ofa_steps_done() + the step's index in the launch): flag values only grow, so nothing needs resetting between launches. */
int ofa_num_buckets(const ofa_ctx* ctx);
int ofa_bucket_span(const ofa_ctx* ctx, int bucket, size_t* offset, size_t* count);   /* elements */
void* ofa_grad_buffer(const ofa_ctx* ctx);
int* ofa_ext_ready_flags(const ofa_ctx* ctx);
int* ofa_ext_done_flags(const ofa_ctx* ctx);
/* The communication side itself, for hosts without their own (no counterpart in the reference): one NCCL communicator per
 * context, looked up at run time (environment OFA_NCCL_LIB = path of libnccl.so.2, else the NCCL the process already holds),
 * never linked. Rank 0 obtains a 128-byte id and hands it to the other ranks by its own means; every rank calls ofa_dp_init
 * (cfg.ext_sync = 1, cfg.dp_world = world) before its first launch. Per launch: ofa_launch(ctx, n); ofa_dp_enqueue(ctx, n) -
 * in this order, a queued stream wait must never precede the kernel that satisfies it - then ofa_dp_wait instead of ofa_wait.
 * ofa_dp_wait returns OFA_OK only when the kernels of ALL ranks ran to the end: the rank whose kernel stopped early returns
 * that failure after releasing its queued waits (ofa_dp_cancel), the others OFA_DEVICE_ABORT. comm_timeout_ms bounds the drain
 * of the communication stream and the status exchange (a missing rank gives OFA_TIMEOUT, not a hang of the host). */
int ofa_dp_unique_id(void* out128);
int ofa_dp_init(ofa_ctx* ctx, const void* id128, int rank, int world);
int ofa_dp_enqueue(ofa_ctx* ctx, int nsteps);
int ofa_dp_cancel(ofa_ctx* ctx);
int ofa_dp_finish(ofa_ctx* ctx, int timeout_ms);
int ofa_dp_wait(ofa_ctx* ctx, int timeout_ms, int comm_timeout_ms, ofa_status_t* status);
void ofa_dp_shutdown(ofa_ctx* ctx);                 /* also done by ofa_destroy */

/* ---- task level -------------------------------------------------------------------------------------------------- */
enum {  /* task kinds, = TaskKind of the device code */
  OFA_TK_DATA = 0, OFA_TK_EMBED, OFA_TK_LN_FWD, OFA_TK_GEMM, OFA_TK_ATT_FWD, OFA_TK_ATT_PREP, OFA_TK_ATT_BWD, OFA_TK_CE,
  OFA_TK_CE_MEAN, OFA_TK_LN_BWD, OFA_TK_LN_DG, OFA_TK_EMB_WTE, OFA_TK_EMB_WPE, OFA_TK_ADAMW, OFA_TK_BARRIER
};
enum { OFA_GEMM_NN = 0, OFA_GEMM_NT = 1, OFA_GEMM_TN = 2 };
enum { OFA_EPI_STORE = 0, OFA_EPI_RES = 1, OFA_EPI_GELU = 2, OFA_EPI_DGELU = 3, OFA_EPI_F32 = 4,
       OFA_EPI_DR = 5 /* C = acc and p[4][b,h,t] = sum over head h's columns of C * aux: attention backward's row term fused into the GEMM that produces dO */,
       OFA_EPI_LSE = 6 /* C = acc and p[4][row][N/128] = float2 {max, sum of exponentials} of each 128-column tile of the stored row, in the log2 domain: softmax partials of the LM head (NT layout); an OFA_TK_CE phase given them as its p[3] reads the logits once instead of twice (the reference's cross-entropy makes two passes, llm/elementwise/ew_loss.cuh:19-75) */ };

/* One phase = ntasks independent block-sized tasks (PhaseDesc, ofa.cu:89-95). Pointers are DEVICE pointers obtained
 * from ofa_dev_alloc. For GEMM phases ntasks/tiles are derived from M,N,K and the TMA descriptors are built here. */
typedef struct {
  int kind, layout, epi, accumulate;
  int M, N, K, lda, ldb, ldc, ldaux, nsub;
  void* p[10];              /* GEMM: p[0]=A p[1]=B p[2]=C p[3]=aux (p[4] = row-term output for OFA_EPI_DR); other kinds: the argument order of the device task */
  size_t n;
  int i0, i1, i2;
} ofa_phase;

typedef struct { int vocab, d_model, n_layer, n_head, ctx_len, batch; } ofa_dims;

int ofa_dev_alloc(void** p, size_t bytes);          /* zero-filled */
int ofa_dev_free(void* p);
int ofa_h2d(void* dst, const void* src, size_t bytes);
int ofa_d2h(void* dst, const void* src, size_t bytes);
/* Runs phases[0..nph) as a chain (phase i waits for phase i-1; phase 0 of repeat r waits for the last phase of r-1),
 * `repeats` times, in one persistent launch on all SMs. ms = CUDA-event time of the launch. AdamW phases use `adam`
 * = {lr, beta1, beta2, eps, wd, grad_scale} with optimizer step r+1. */
int ofa_run_phases(int dtype, const ofa_dims* dims, const ofa_phase* phases, int nph, int repeats, const float* adam,
                   float* ms, ofa_status_t* status);
/* Test hook: with seed != 0 every phase uploaded afterwards (by ofa_launch or ofa_run_phases, training and serving graphs) hands
 * its tasks out in a pseudo-randomly permuted order; 0 restores the natural order. Every result must be bit-identical either
 * way: the reference checks its task libraries the same way (llm/gemm/test_gemm.cu:20-49, llm/attention/test_attention.cu:45-77,
 * llm/decode/test_decode.cu:135-158 pull tasks in shuffled orders). Process-global, not for production use. */
void ofa_debug_set_task_shuffle(unsigned seed);

/* ---- allocation-free entry point ------------------------------------------------------------------------------------
 * No counterpart in the reference (its program allocates everything up front in main()). LayerNorm backward for the bf16
 * path (d_model 768): dx = LN'(dy) [+ dres], dgamma (=|+=) column sums - the same arithmetic as the TK_LN_BWD + TK_LN_DG
 * phases - as two ordinary kernel launches on `stream` (a cudaStream_t, or NULL) that call no cudaMalloc / cudaFree and no
 * allocating library routine. It is for hosts that cannot allocate device memory on this path: processes whose GPU memory
 * belongs to another allocator's pool, and loops that share the device with a resident persistent kernel, where the
 * device-wide synchronisation of an allocation would stall that kernel. The dgamma partials live in a fixed device array
 * (about 6 MB per GPU, kept until exit), so n_rows <= ofa_noalloc_max_rows() (32768); larger sizes return OFA_BAD_ARGUMENT
 * and launch nothing. All pointers are device pointers supplied by the caller (bf16 for dx, dy, x, gamma, dres; dres may
 * be NULL). The array is shared by every call and keeps the last call's partials (each call overwrites all it reads, so
 * nothing needs clearing): calls that overlap on the GPU race and must be serialised by the caller. The first call on a
 * device resolves the array's address with that device current; issue it before any stream capture begins. */
int ofa_ln_bwd_noalloc(void* dx, float* dgamma, const void* dy, const void* x, const float* mean, const float* rstd,
                       const void* gamma, const void* dres, int n_rows, int d_model, int accumulate, void* stream);
int ofa_noalloc_max_rows(void);
const char* ofa_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
