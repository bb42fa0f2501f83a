// Contexts: creation, the default context per device, options, tracing read-out.
#include <mutex>

#include "context.cuh"

namespace orca {

static thread_local Ctx *g_cur = nullptr;

static int create_ctx(Ctx **out) {
  Ctx *c = new Ctx();
  ORCA_CUDA(cudaGetDevice(&c->device));
  int sms = 0;
  ORCA_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device));
  if (sms > 0) c->sm_count = sms;
  ORCA_CUDA(cudaStreamCreateWithFlags(&c->aux, cudaStreamNonBlocking));
  ORCA_CUDA(cudaStreamCreateWithFlags(&c->idx, cudaStreamNonBlocking));
  ORCA_CUDA(cudaStreamCreateWithFlags(&c->lane1, cudaStreamNonBlocking));
  ORCA_CUDA(cudaStreamCreateWithFlags(&c->copy, cudaStreamNonBlocking));
  for (int q = 0; q < Ctx::kStageSlots; ++q) ORCA_CUDA(cudaEventCreateWithFlags(&c->ev_slot[q], cudaEventDisableTiming));
  cudaEvent_t *evs[] = {&c->fork, &c->join, &c->ev_in, &c->ev_flags, &c->ev_o1, &c->ev_g2, &c->ev_state,
                        &c->ev_idx[0], &c->ev_idx[1], &c->ev_done[0], &c->ev_done[1]};
  for (cudaEvent_t *e : evs) ORCA_CUDA(cudaEventCreateWithFlags(e, cudaEventDisableTiming));
  ORCA_CUDA(cudaMalloc(&c->d_words, CTX_WORDS * sizeof(int32_t)));
  ORCA_CUDA(cudaMemset(c->d_words, 0, CTX_WORDS * sizeof(int32_t)));
  *out = c;
  return ORCA_OK;
}

static void destroy_ctx(Ctx *c) {
  if (c == nullptr) return;
  int prev = -1;
  cudaGetDevice(&prev);
  if (c->device >= 0) cudaSetDevice(c->device);
  if (c->aux) cudaStreamSynchronize(c->aux);
  if (c->idx) cudaStreamSynchronize(c->idx);
  if (c->lane1) cudaStreamSynchronize(c->lane1);
  if (c->copy) cudaStreamSynchronize(c->copy);
  for (cudaEvent_t e : c->ev_slot)
    if (e) cudaEventDestroy(e);
  cudaEvent_t evs[] = {c->fork, c->join, c->ev_in, c->ev_flags, c->ev_o1, c->ev_g2, c->ev_state, c->ev_idx[0],
                       c->ev_idx[1], c->ev_done[0], c->ev_done[1]};
  for (cudaEvent_t e : evs)
    if (e) cudaEventDestroy(e);
  for (cudaEvent_t e : c->trace.ev) cudaEventDestroy(e);
  for (cudaEvent_t e : c->prof.ev) cudaEventDestroy(e);
  if (c->aux) cudaStreamDestroy(c->aux);
  if (c->idx) cudaStreamDestroy(c->idx);
  if (c->lane1) cudaStreamDestroy(c->lane1);
  if (c->copy) cudaStreamDestroy(c->copy);
  if (c->d_words) cudaFree(c->d_words);
  if (prev >= 0) cudaSetDevice(prev);
  delete c;
}

Ctx *default_ctx() {
  constexpr int kMaxDevices = 64;
  static Ctx *of_device[kMaxDevices] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (of_device[dev] == nullptr) {
    Ctx *c = nullptr;
    if (create_ctx(&c) != ORCA_OK) return nullptr;
    of_device[dev] = c;
  }
  return of_device[dev];
}

Ctx *cur() { return g_cur != nullptr ? g_cur : default_ctx(); }

CtxScope::CtxScope(Ctx *c) : prev(g_cur) { g_cur = c; }
CtxScope::~CtxScope() { g_cur = prev; }

bool dependent_launch_enabled() {
  Ctx *c = cur();
  return c == nullptr || c->dependent_launch;
}

int Tracer::mark(int phase, cudaStream_t s) {
  if (!on) return ORCA_OK;
  if (used == ev.size()) {
    cudaEvent_t e;
    ORCA_CUDA(cudaEventCreate(&e));
    ev.push_back(e);
    phase_of.push_back(-1);
  }
  phase_of[used] = phase;
  ORCA_CUDA(cudaEventRecord(ev[used++], s));
  return ORCA_OK;
}

static const char *kPhaseNames[PH_COUNT] = {"prep", "sample_top", "find_uncached", "sample_l1", "last_occurrence_l1",
                                            "attn_query_l1", "attn_gather_l1", "attn_output_l1", "set_flags",
                                            "attn_query_l2", "attn_gather_l2", "attn_output_l2", "score",
                                            "last_occurrence_msg", "message_store", "gru_update"};

static Ctx *resolve(orca_ctx_t *ctx) { return ctx != nullptr ? reinterpret_cast<Ctx *>(ctx) : default_ctx(); }

}  // namespace orca

using namespace orca;

extern "C" {

int orca_ctx_create(orca_ctx_t **out) {
  ORCA_CHECK_ARG(out != nullptr);
  Ctx *c = nullptr;
  int rc = create_ctx(&c);
  if (rc != ORCA_OK) {
    destroy_ctx(c);
    return rc;
  }
  *out = reinterpret_cast<orca_ctx_t *>(c);
  return ORCA_OK;
}

int orca_ctx_destroy(orca_ctx_t *ctx) {
  destroy_ctx(reinterpret_cast<Ctx *>(ctx));
  return ORCA_OK;
}

int orca_ctx_set(orca_ctx_t *ctx, int32_t option, int64_t value) {
  Ctx *c = resolve(ctx);
  if (c == nullptr) return set_error(ORCA_E_CUDA, "orca_ctx_set: no context for the current device");
  switch (option) {
    case ORCA_OPT_PROJECTION_MODE:
      ORCA_CHECK_ARG(value == 0 || value == 1);
      c->projection_mode = (int)value;
      break;
    case ORCA_OPT_OVERLAP: c->overlap = value != 0; break;
    case ORCA_OPT_DEPENDENT_LAUNCH: c->dependent_launch = value != 0; break;
    case ORCA_OPT_LOOKAHEAD: c->lookahead = value != 0; break;
    case ORCA_OPT_WAIT_LIMIT:
      ORCA_CHECK_ARG(value > 0);
      c->wait_limit = (long long)value;
      break;
    case ORCA_OPT_TRACE:
      c->trace.on = value != 0;
      c->trace.used = 0;
      break;
    default: return set_error(ORCA_E_BADARG, "orca_ctx_set: unknown option %d", option);
  }
  return ORCA_OK;
}

int orca_ctx_set_status_word(orca_ctx_t *ctx, int32_t *d_status) {
  Ctx *c = resolve(ctx);
  if (c == nullptr) return set_error(ORCA_E_CUDA, "orca_ctx_set_status_word: no context for the current device");
  c->status_word = d_status;
  return ORCA_OK;
}

int orca_ctx_last_parity(orca_ctx_t *ctx) {
  Ctx *c = resolve(ctx);
  return c != nullptr ? c->last_parity : 0;
}

int orca_trace_phases(void) { return PH_COUNT; }
const char *orca_trace_phase_name(int32_t phase) {
  return (phase >= 0 && phase < PH_COUNT) ? kPhaseNames[phase] : "";
}

int orca_trace_read(orca_ctx_t *ctx, double *h_ms_per_phase) {
  ORCA_CHECK_ARG(h_ms_per_phase);
  Ctx *c = resolve(ctx);
  if (c == nullptr) return set_error(ORCA_E_CUDA, "orca_trace_read: no context for the current device");
  Tracer &t = c->trace;
  for (int i = 0; i < PH_COUNT; ++i) h_ms_per_phase[i] = 0.0;
  for (size_t i = 1; i < t.used; ++i) {
    const int ph = t.phase_of[i];
    if (ph < 0) continue;  // first event of a batch
    ORCA_CUDA(cudaEventSynchronize(t.ev[i]));
    float ms = 0.f;
    ORCA_CUDA(cudaEventElapsedTime(&ms, t.ev[i - 1], t.ev[i]));
    h_ms_per_phase[ph] += ms;
  }
  t.used = 0;
  return ORCA_OK;
}

int orca_attn_gather_profile(orca_ctx_t *ctx, int32_t enable, void *d_counters) {
  Ctx *c = resolve(ctx);
  if (c == nullptr) return set_error(ORCA_E_CUDA, "orca_attn_gather_profile: no context for the current device");
  c->prof.on = enable != 0;
  c->prof.d_counters = (unsigned long long *)d_counters;
  c->prof.used = 0;
  return ORCA_OK;
}

int orca_attn_gather_profile_read(orca_ctx_t *ctx, double *h_ms_total, int64_t *h_launches) {
  ORCA_CHECK_ARG(h_ms_total && h_launches);
  Ctx *c = resolve(ctx);
  if (c == nullptr) return set_error(ORCA_E_CUDA, "orca_attn_gather_profile_read: no context for the current device");
  GatherProfile &p = c->prof;
  double total = 0.0;
  for (size_t i = 0; i + 1 < p.used; i += 2) {
    ORCA_CUDA(cudaEventSynchronize(p.ev[i + 1]));
    float ms = 0.f;
    ORCA_CUDA(cudaEventElapsedTime(&ms, p.ev[i], p.ev[i + 1]));
    total += ms;
  }
  *h_ms_total = total;
  *h_launches = (int64_t)(p.used / 2);
  p.used = 0;
  return ORCA_OK;
}

}  // extern "C"
