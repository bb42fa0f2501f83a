// Per-caller context of the library: the auxiliary streams and events of the batch pipeline, the
// switches that used to be process-wide (projection mode, overlap, dependent launch, look-ahead,
// wait limit, tracing), the status word the projection kernels report to, and a few zeroed device
// words (work tickets of the gather kernel).  A model descriptor carries its context; the stand-alone
// kernel entry points use the default context of the current device.
#pragma once

#include <vector>

#include "common.cuh"

namespace orca {

enum Phase { PH_PREP, PH_SAMPLE_TOP, PH_UNCACHED, PH_SAMPLE_L1, PH_LAST_OCC_L1, PH_QUERY_L1, PH_GATHER_L1,
             PH_OUTPUT_L1, PH_FLAGS, PH_QUERY_L2, PH_GATHER_L2, PH_OUTPUT_L2, PH_SCORE, PH_LAST_OCC_MSG,
             PH_MESSAGE, PH_GRU, PH_COUNT };

struct Tracer {
  bool on = false;
  std::vector<cudaEvent_t> ev;        // events of the traced batches, in recording order
  std::vector<int> phase_of;          // phase that ENDS at event i (or -1 for a batch's first event)
  size_t used = 0;
  int mark(int phase, cudaStream_t s);
};

struct GatherProfile {
  bool on = false;
  unsigned long long *d_counters = nullptr;
  std::vector<cudaEvent_t> ev;   // pairs (start, stop)
  size_t used = 0;
};

constexpr int CTX_WORDS = 256;            // zeroed device words owned by a context
constexpr int CTX_TICKET_MAIN = 0;        // gather-kernel tickets: {next row, finished warps} per lane of work
constexpr int CTX_TICKET_SIDE = 2;

struct Ctx {
  int device = -1;
  int sm_count = 148;
  // switches
  int projection_mode = 0;                // 0 = tensor cores (bf16 head/tail split), 1 = fp32 SIMT tiles
  bool overlap = true;                    // raw-message / GRU chain on the auxiliary stream
  bool dependent_launch = true;           // programmatic stream serialisation
  bool lookahead = true;                  // index work of a batch on its own stream, ahead of the chain
  long long wait_limit = 2000000000ll;    // SM clocks a device-side wait may spin before it gives up
  int32_t *status_word = nullptr;         // where the projection kernels report a wait that gave up
  // streams and events of the batch pipeline (created with the context)
  static constexpr int kStageSlots = 4;   // batches the staging ring of orca_tgn_eval_epoch holds
  cudaStream_t aux = nullptr, idx = nullptr, lane1 = nullptr, copy = nullptr;
  cudaEvent_t ev_slot[kStageSlots] = {nullptr, nullptr, nullptr, nullptr};
  bool slot_used[kStageSlots] = {false, false, false, false};
  long long stage_seq = 0;
  cudaEvent_t fork = nullptr, join = nullptr, ev_in = nullptr, ev_flags = nullptr;
  cudaEvent_t ev_o1 = nullptr, ev_g2 = nullptr, ev_state = nullptr;
  cudaEvent_t ev_idx[2] = {nullptr, nullptr}, ev_done[2] = {nullptr, nullptr};
  bool done_recorded[2] = {false, false}, state_recorded = false, g2_recorded = false;
  long long seq = 0;                      // budgeted two-layer batches enqueued through this context
  int parity = 0;                         // buffer parity of the batch being enqueued (kept between the
  long long base1 = 0, base_msg = 0;      // two phases of a sharded batch, like its record bases
  long long xseq = 0;                     // and its sequence number in the ranks' flag words)
  int last_parity = 0;
  int layout_b = 0, layout_u = 0, layout_k = 0;   // workspace layout of the last budgeted batch
  const void *layout_ws = nullptr;
  int last_batch_launches = 0;
  int32_t *d_words = nullptr;             // CTX_WORDS zeroed int32
  Tracer trace;
  GatherProfile prof;
};

// the context in effect for the calling thread: the one of the running batch entry point, else the
// default context of the current device (created on first use; nullptr if that fails)
Ctx *cur();
Ctx *default_ctx();
struct CtxScope {
  Ctx *prev;
  explicit CtxScope(Ctx *c);
  ~CtxScope();
};

}  // namespace orca
