// Command-line host for libofa_b200.so: what main() of the reference's megakernel program (llm/b200/megakernel/ofa.cu:394-766)
// becomes when its body is replaced by calls into include/ofa_b200.h. Same flags for the path this library covers, same
// files, same report lines; Doom, the dashboard and the vocabulary-to-text printing are not part of the library.
//
//   ofa_cli --preset gpt_s --split b200 --steps 4000 --data tokens.u32 --starts starts.u32 --init init_flat.f32 \
//           --prompt prompt.txt --answer-len 256 --temp 0.8 --loss-out loss.txt --text-out tokens.txt --dump-w w.f32
//
// Without --data a uniform synthetic token stream is generated (the flag --synthetic-seed picks it); without --init the
// weights are drawn by a xorshift normal generator (scale 0.02, residual projections 0.02/sqrt(2L), gains 1), which is NOT the
// PyTorch recipe of the oracle - parity runs pass --init.
#include "../../include/ofa_b200.h"
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

namespace {

template <class T> bool read_file(const std::string& path, std::vector<T>& out) {
  FILE* f = fopen(path.c_str(), "rb");
  if (!f) { fprintf(stderr, "cannot open %s\n", path.c_str()); return false; }
  fseek(f, 0, SEEK_END); const long bytes = ftell(f); fseek(f, 0, SEEK_SET);
  out.resize((size_t)bytes / sizeof(T));
  const size_t got = fread(out.data(), sizeof(T), out.size(), f);
  fclose(f);
  return got == out.size();
}
template <class T> bool write_file(const std::string& path, const std::vector<T>& v) {
  FILE* f = fopen(path.c_str(), "wb");
  if (!f) { fprintf(stderr, "cannot write %s\n", path.c_str()); return false; }
  const size_t put = fwrite(v.data(), sizeof(T), v.size(), f);
  fclose(f);
  return put == v.size();
}
struct Xorshift {
  uint64_t s;
  uint64_t next() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return s; }
  double uniform() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }
  float normal() { const double u = std::max(uniform(), 1e-300), v = uniform(); return (float)(std::sqrt(-2.0 * std::log(u)) * std::cos(6.283185307179586 * v)); }
};
int fail(ofa_ctx* ctx, const char* what) {
  fprintf(stderr, "%s: %s\n", what, ofa_last_error(ctx));
  if (ctx) ofa_destroy(ctx);
  return 1;
}
void usage() {
  printf("ofa_cli [--preset gpt_s|tiny] [--tied] [--steps N] [--sched-steps N] [--split b200|none] [--infer-sms N] [--doom-sms N]\n"
         "        [--train-sms N] [--data file.u32] [--starts file.u32] [--init flat.f32] [--seed N] [--synthetic-seed N]\n"
         "        [--prompt ids.txt] [--answer-len N] [--temp T] [--no-opt] [--loss-out file] [--text-out file]\n"
         "        [--dump-w flat.f32] [--dump-grads flat.f32] [--device N]\n"
         "flags and file formats are those of the reference's megakernel program for the training + serving path\n");
}

}  // namespace

int main(int argc, char** argv) {
  int steps = 100, sched_steps = 4000, infer_sms = 0, doom_sms = 0, train_sms = -1, nopt = 0, answer_len = 0, device = 0, tied = -1;
  std::string preset = "gpt_s", split_mode = getenv("OFA_SPLIT") ? getenv("OFA_SPLIT") : "";
  std::string data_path, init_path, starts_path, dump_grads, dump_w, loss_out, text_out, prompt_path;
  float temp = 0.8f; unsigned long long seed = 1234, synth_seed = 0;
  for (int i = 1; i < argc; i++) {
    auto is = [&](const char* s) { return !strcmp(argv[i], s) && i + 1 < argc; };
    if (!strcmp(argv[i], "--help") || !strcmp(argv[i], "-h")) { usage(); return 0; }
    else if (is("--steps")) steps = atoi(argv[++i]); else if (is("--sched-steps")) sched_steps = atoi(argv[++i]);
    else if (is("--data")) data_path = argv[++i]; else if (is("--init")) init_path = argv[++i]; else if (is("--starts")) starts_path = argv[++i];
    else if (is("--dump-grads")) dump_grads = argv[++i]; else if (is("--dump-w")) dump_w = argv[++i]; else if (is("--loss-out")) loss_out = argv[++i];
    else if (is("--infer-sms")) infer_sms = atoi(argv[++i]); else if (is("--doom-sms")) doom_sms = atoi(argv[++i]);
    else if (is("--train-sms")) train_sms = atoi(argv[++i]); else if (is("--split")) split_mode = argv[++i];
    else if (is("--seed")) seed = strtoull(argv[++i], nullptr, 10); else if (is("--synthetic-seed")) synth_seed = strtoull(argv[++i], nullptr, 10);
    else if (is("--temp")) temp = (float)atof(argv[++i]); else if (is("--text-out")) text_out = argv[++i]; else if (is("--prompt")) prompt_path = argv[++i];
    else if (is("--answer-len")) answer_len = atoi(argv[++i]); else if (is("--preset")) preset = argv[++i]; else if (is("--device")) device = atoi(argv[++i]);
    else if (!strcmp(argv[i], "--no-opt")) nopt = 1; else if (!strcmp(argv[i], "--tied")) tied = 1;
    else { fprintf(stderr, "unknown or incomplete flag %s\n", argv[i]); usage(); return 2; }
  }
  ofa_config cfg;
  if (ofa_default_config(&cfg, preset.c_str()) != OFA_OK) { fprintf(stderr, "unknown preset %s\n", preset.c_str()); return 2; }
  if (tied >= 0) cfg.tied_head = tied;
  cfg.device = device; cfg.sched_steps = sched_steps; cfg.data_seed = seed; cfg.decode_seed = seed;
  if (nopt) cfg.mode = OFA_MODE_NO_OPT;
  // the partition: explicit flags > --split / OFA_SPLIT > none (train only). "b200" = 24 serving, 8 reserved, 116 training SMs
  // (ofa.cu:384-391); the SMs the reference gives to Doom are reserved and idle here.
  if (infer_sms == 0 && !split_mode.empty() && split_mode != "none") {
    if (split_mode != "b200" && split_mode != "auto") { fprintf(stderr, "--split must be auto|b200|none\n"); return 2; }
    infer_sms = 24; doom_sms = 8; if (train_sms < 0) train_sms = 116;
  }
  cfg.infer_sms = infer_sms; cfg.reserved_sms = infer_sms > 0 ? doom_sms : 0; cfg.train_sms = train_sms > 0 ? train_sms : 0;
  cfg.use_decode = infer_sms > 0 ? 1 : 0;
  cfg.temperature = temp; cfg.answer_len = answer_len; cfg.decode_out_cap = 1 << 20;
  if (!prompt_path.empty()) {
    FILE* f = fopen(prompt_path.c_str(), "r"); int x; cfg.n_prompt = 0;
    while (f && cfg.n_prompt < 32 && fscanf(f, "%d", &x) == 1) cfg.prompt[cfg.n_prompt++] = x;
    if (f) fclose(f);
  }
  if (cfg.use_decode && cfg.n_prompt == 0) { cfg.n_prompt = 1; cfg.prompt[0] = 0; }

  ofa_ctx* ctx = nullptr;
  if (ofa_create(&cfg, &ctx) != OFA_OK) return fail(nullptr, "ofa_create");
  const size_t NP = ofa_num_params(ctx);
  printf("model %s: V %d D %d L %d H %d T %d B %d (%s head), %zu parameters; SMs: serve %d, reserved %d, train %s\n", preset.c_str(), cfg.vocab,
         cfg.d_model, cfg.n_layer, cfg.n_head, cfg.ctx_len, cfg.batch, cfg.tied_head ? "tied" : "untied", NP, cfg.infer_sms, cfg.reserved_sms,
         cfg.train_sms > 0 ? std::to_string(cfg.train_sms).c_str() : "all others");

  // ---- weights: --init file (flat fp32 in the library's parameter order), or the built-in generator
  std::vector<float> w;
  if (!init_path.empty()) {
    if (!read_file(init_path, w)) return fail(ctx, "--init");
    if (w.size() != NP) { fprintf(stderr, "%s holds %zu values, the model has %zu parameters\n", init_path.c_str(), w.size(), NP); ofa_destroy(ctx); return 1; }
  } else {
    w.assign(NP, 0.f);
    Xorshift rng{seed * 2654435761ull + 88172645463325252ull};
    const float s0 = 0.02f, sres = 0.02f / std::sqrt(2.f * (float)cfg.n_layer);
    auto fill = [&](const std::string& name, float scale, bool ones) {
      size_t off = 0, n = 0;
      if (ofa_param_span(ctx, name.c_str(), &off, &n) != OFA_OK) return;
      for (size_t i = 0; i < n; i++) w[off + i] = ones ? 1.f : scale * rng.normal();
    };
    fill("wte", s0, false); fill("wpe", s0, false);
    if (!cfg.tied_head) fill("lm_head", s0, false);
    for (int l = 0; l < cfg.n_layer; l++) {
      const std::string p = "L" + std::to_string(l) + ".";
      fill(p + "g1", 0, true); fill(p + "Wqkv", s0, false); fill(p + "Wo", sres, false); fill(p + "g2", 0, true); fill(p + "Wup", s0, false); fill(p + "Wdn", sres, false);
    }
    fill("gf", 0, true);
  }
  if (ofa_load_weights(ctx, w.data(), NP) != OFA_OK) return fail(ctx, "ofa_load_weights");

  // ---- tokens and window starts
  std::vector<uint32_t> tokens, starts;
  if (!data_path.empty()) { if (!read_file(data_path, tokens)) return fail(ctx, "--data"); }
  else {
    tokens.resize((size_t)1 << 22);
    Xorshift rng{synth_seed * 0x9E3779B97F4A7C15ull + 0x2545F4914F6CDD1Dull};
    for (auto& t : tokens) t = (uint32_t)(rng.next() % (uint64_t)cfg.vocab);
    printf("no --data: %zu uniform synthetic token ids\n", tokens.size());
  }
  if (ofa_set_tokens(ctx, tokens.data(), tokens.size()) != OFA_OK) return fail(ctx, "ofa_set_tokens");
  if (!starts_path.empty()) {
    if (!read_file(starts_path, starts)) return fail(ctx, "--starts");
    if (ofa_set_starts(ctx, starts.data(), starts.size() / (size_t)cfg.batch) != OFA_OK) return fail(ctx, "ofa_set_starts");
  }

  // ---- the launch and the 200 ms poll (ofa.cu:710-716)
  const auto tw0 = std::chrono::steady_clock::now();
  if (ofa_launch(ctx, steps) != OFA_OK) return fail(ctx, "ofa_launch");
  ofa_status_t st; int rc;
  while ((rc = ofa_wait(ctx, 200, &st)) == OFA_TIMEOUT) {
    ofa_live_t lv;
    if (ofa_live(ctx, &lv) == OFA_OK) { printf("\r  step %u / %d  loss %.4f  decode tokens %u   ", lv.steps, steps, lv.loss, lv.decode_steps); fflush(stdout); }
  }
  printf("\n");
  if (rc != OFA_OK) {
    if (rc == OFA_DEVICE_ABORT) fprintf(stderr, "device abort: code %d phase %d task %d block %d aux %d\n", st.dev_code, st.phase, st.task, st.block, st.aux);
    return fail(ctx, "ofa_wait");
  }
  const double wall = std::chrono::duration<double>(std::chrono::steady_clock::now() - tw0).count();
  const double ms = ofa_last_launch_ms(ctx);

  // ---- results (the report of ofa.cu:722-756)
  std::vector<float> loss(steps); std::vector<unsigned long long> sd(steps);
  if (ofa_read_losses(ctx, loss.data(), steps) != OFA_OK || ofa_read_step_times(ctx, sd.data(), steps) != OFA_OK) return fail(ctx, "read results");
  printf("kernel time %.3f s (event) / %.3f s (wall incl. launch)\n", ms / 1e3, wall);
  const int w0 = std::min(steps - 1, 3); const int nstep_t = steps - 1 - w0;
  if (nstep_t > 0) {
    const double train_s = (double)(sd[steps - 1] - sd[w0]) * 1e-9;
    std::vector<double> dts; for (int s = w0 + 1; s < steps; s++) dts.push_back((double)(sd[s] - sd[s - 1]) * 1e-6);
    std::sort(dts.begin(), dts.end());
    printf("steady state: %.2f ms/step (median %.2f) -> %.0f tok/s;  4,000 steps = %.1f s\n", train_s * 1e3 / nstep_t, dts[dts.size() / 2],
           (double)cfg.batch * cfg.ctx_len * nstep_t / train_s, 4000 * train_s / nstep_t);
  }
  printf("loss: step0 %.4f", loss[0]);
  for (int s : {1, 2, 5, 10, 20, 50, 100, 200, 500, 1000, 2000, 3000, 3999}) if (s < steps) printf("  s%d %.4f", s, loss[s]);
  printf("\n");
  if (!loss_out.empty()) { FILE* f = fopen(loss_out.c_str(), "w"); if (f) { for (int s = 0; s < steps; s++) fprintf(f, "%d %.6f\n", s, loss[s]); fclose(f); } }
  {  // busy time by phase kind (all steps, block-seconds; % of training busy time)
    const int nph = ofa_num_phases(ctx);
    std::vector<std::pair<std::string, double>> grp; double tot = 0;
    for (int i = 0; i < nph; i++) {
      char name[64]; int kind = 0, nt = 0; unsigned long long busy = 0;
      if (ofa_phase_info(ctx, i, name, sizeof name, &kind, &nt, &busy) != OFA_OK) continue;
      std::string nme = name; const size_t sp = nme.find(' ');
      const std::string key = (nme[0] == 'L' && sp != std::string::npos && isdigit((unsigned char)nme[1])) ? nme.substr(sp + 1) : nme;
      bool found = false; for (auto& g : grp) if (g.first == key) { g.second += (double)busy; found = true; }
      if (!found) grp.push_back({key, (double)busy});
      tot += (double)busy;
    }
    printf("\nbusy time by phase kind (all steps, block-seconds; %% of train busy):\n");
    for (auto& g : grp) printf("  %-18s %8.3f s  %5.1f%%\n", g.first.c_str(), g.second * 1e-9, tot > 0 ? 100 * g.second / tot : 0.0);
  }
  if (cfg.use_decode) {
    const int dstep = ofa_decode_steps(ctx);
    const double span = steps > 1 ? (double)(sd[steps - 1] - sd[0]) * 1e-9 + 1e-9 : ms * 1e-3;
    printf("decode: %d tokens generated during %.2f s of training -> %.0f tok/s\n", dstep, span, dstep / span);
    std::vector<int> ring((size_t)cfg.decode_out_cap, -1);
    const int cnt = std::min(dstep, cfg.decode_out_cap);
    if (ofa_read_decode_tokens(ctx, ring.data(), ring.size()) == OFA_OK) {
      long gen = 0, answers = 0;
      for (int i = 0; i < cnt; i++) { const int id = ring[i]; if (id == OFA_OUT_RESTART) answers++; else if (id >= 0 && id < OFA_OUT_RESTART) gen++; }
      if (answer_len > 0)
        printf("decode answers: %ld answers (%d prompt tokens + %d sampled each), %ld sampled tokens -> %.0f tok/s sampled (prompt steps excluded)\n",
               answers, cfg.n_prompt, answer_len, gen, gen / span);
      if (!text_out.empty()) { FILE* f = fopen(text_out.c_str(), "w"); if (f) { for (int i = 0; i < cnt; i++) fprintf(f, "%d ", ring[i]); fclose(f); } }
      printf("first sampled token ids:"); for (int i = 0; i < std::min(cnt, 40); i++) printf(" %d", ring[i]); printf("\n");
    }
  }
  if (!dump_grads.empty()) { std::vector<float> h(NP); if (ofa_read_grads(ctx, h.data(), NP) == OFA_OK && write_file(dump_grads, h)) printf("wrote grads %s\n", dump_grads.c_str()); }
  if (!dump_w.empty()) { std::vector<float> h(NP); if (ofa_read_weights(ctx, h.data(), NP) == OFA_OK && write_file(dump_w, h)) printf("wrote weights %s\n", dump_w.c_str()); }
  ofa_destroy(ctx);
  return 0;
}
