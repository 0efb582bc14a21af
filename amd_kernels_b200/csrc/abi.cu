// Library identity, workspace carving and the whole-layer entry points.
#include "common.cuh"

namespace b200moe {

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Workspace {
  float* w;               // [T][4]
  int32_t* ids;           // [T][4]
  int32_t* sorted_ids;    // [R]
  float* sorted_w;        // [R]
  int32_t* block_expert;  // [R/bm]
  int32_t* num_valid;     // [2]
  int32_t* scratch;       // permute chunk counts
  uint8_t* xq_sorted;     // [R][3072]
  uint8_t* sfx;           // [R/bm][48][512]
  uint8_t* hq;            // [R][384]
  uint8_t* sfh;           // [R/bm][6][512]
  int32_t* done;          // [R/bm] GEMM1 tiles finished per row block (one-launch GEMM1+GEMM2)
  // only with the router inside the call (b200moe_forward_x):
  float* partials;        // [S][T][E] split-K logit partials
  uint8_t* q4;            // [T][3072] row-major MXFP4 codes of x
  uint8_t* s4;            // [T][192] their scales
  size_t bytes;
  int bm;
  int64_t rows;
};

int dispatch_rows_done(const uint8_t* codes, const uint8_t* scales, const int32_t* sorted_ids, const int32_t* num_valid,
                       int64_t tokens, int bm, int by_pair, int64_t max_rows, uint8_t* xq_sorted, uint8_t* sfx,
                       int32_t* done, void* stream);
int prep_small(const float* partials, int64_t stride_t, int64_t stride_s, int splits, const float* bias, int64_t tokens,
               int num_experts, int mode, float scale, int bm, float* out_w, int32_t* out_ids, int32_t* sorted_ids,
               float* sorted_w, int32_t* block_expert, int32_t* num_valid, const void* x_bf16, const uint8_t* q4,
               const uint8_t* s4, int64_t max_rows, uint8_t* xq_sorted, uint8_t* sfx, int32_t* done, int n_done,
               void* stream);
int quant_rows(const void* x_bf16, int64_t tokens, uint8_t* codes, uint8_t* scales, void* stream);
int set_wait_limit_routed(unsigned long long ns);
int set_wait_limit_shared(unsigned long long ns);
int set_wait_limit_pair(unsigned long long ns);
int set_wait_limit_router(unsigned long long ns);
int set_wait_limit_ep_sync(unsigned long long ns);

static Workspace carve(uint8_t* base, int64_t tokens, int num_experts, bool with_router = false) {
  Workspace ws{};
  ws.bm = b200moe_block_rows(tokens);
  ws.rows = b200moe_max_sorted_rows(tokens, ws.bm, num_experts);
  const size_t blocks = static_cast<size_t>(ws.rows / ws.bm);
  size_t off = 0;
  auto take = [&](size_t n) {
    uint8_t* p = base ? base + off : nullptr;
    off = align_up(off + n, 1024);
    return p;
  };
  ws.w = reinterpret_cast<float*>(take(tokens * kTopK * 4));
  ws.ids = reinterpret_cast<int32_t*>(take(tokens * kTopK * 4));
  ws.sorted_ids = reinterpret_cast<int32_t*>(take(ws.rows * 4));
  ws.sorted_w = reinterpret_cast<float*>(take(ws.rows * 4));
  ws.block_expert = reinterpret_cast<int32_t*>(take(blocks * 4));
  ws.num_valid = reinterpret_cast<int32_t*>(take(16));
  ws.scratch = reinterpret_cast<int32_t*>(take(b200moe_permute_scratch_bytes(tokens, num_experts) + 16));
  ws.xq_sorted = take(ws.rows * (kH / 2));
  ws.sfx = take(blocks * (kH / 128) * kAtomBytes);
  ws.hq = take(ws.rows * (kI / 2));
  ws.sfh = take(blocks * (kI / 128) * kAtomBytes);
  ws.done = reinterpret_cast<int32_t*>(take(blocks * 4));
  if (with_router)
    ws.partials = reinterpret_cast<float*>(take(static_cast<size_t>(b200moe_router_splits(tokens)) * tokens * num_experts * 4));
  if (with_router || ws.bm == 128) {  // row-major quantised tokens: the router path always, the logits path at prefill sizes
    ws.q4 = take(tokens * (kH / 2));
    ws.s4 = take(tokens * (kH / 32));
  }
  ws.bytes = off;
  return ws;
}

}  // namespace b200moe

extern "C" int b200moe_version(void) { return 1; }
extern "C" const char* b200moe_arch(void) { return "sm_100a"; }

extern "C" size_t b200moe_workspace_bytes(int64_t tokens, int num_experts) {
  if (tokens < 1 || tokens > B200MOE_MAX_TOKENS || num_experts < 1 || num_experts > b200moe::kMaxE) return 0;
  return b200moe::carve(nullptr, tokens, num_experts).bytes;
}

extern "C" size_t b200moe_workspace_bytes_x(int64_t tokens, int num_experts) {
  if (tokens < 1 || tokens > B200MOE_MAX_TOKENS || num_experts < 1 || num_experts > b200moe::kMaxE) return 0;
  return b200moe::carve(nullptr, tokens, num_experts, true).bytes;
}

extern "C" int b200moe_set_wait_limit_ns(uint64_t ns) {
  if (ns == 0) return B200MOE_E_ARG;
  int r = b200moe::set_wait_limit_routed(ns);
  if (!r) r = b200moe::set_wait_limit_shared(ns);
  if (!r) r = b200moe::set_wait_limit_pair(ns);
  if (!r) r = b200moe::set_wait_limit_router(ns);
  if (!r) r = b200moe::set_wait_limit_ep_sync(ns);
  return r;
}

namespace b200moe {
constexpr int64_t kSmallTokens = 32;  // up to here a layer call is three launches: preparation, both GEMMs, reduce
// sorted, gathered, quantised rows are in the workspace: the grouped GEMMs and the reduce
static int experts_and_reduce(const b200moe_weights* w, const Workspace& ws, int64_t tokens, void* slots_bf16,
                              void* out_bf16, int32_t* status, void* stream) {
  const int ne = w->num_experts;
  int r;
  if (tokens <= kSmallTokens) {  // small batches: both grouped GEMMs in one persistent launch (measured faster there only)
    if ((r = b200moe_gemm12(w->w13t, w->w2t, ne, ws.xq_sorted, ws.sfx, ws.block_expert, ws.num_valid, ws.sorted_ids,
                            ws.sorted_w, ws.rows, ws.bm, tokens, ws.hq, ws.sfh, ws.done, slots_bf16, status, stream)))
      return r;
  } else {
    if ((r = b200moe_gemm1_swiglu_quant(w->w13t, ne, ws.xq_sorted, ws.sfx, ws.block_expert, ws.num_valid, ws.rows, ws.bm,
                                        ws.hq, ws.sfh, w->w2t, status, stream)))
      return r;
    if ((r = b200moe_gemm2_weighted(w->w2t, ne, ws.hq, ws.sfh, ws.block_expert, ws.num_valid, ws.sorted_ids, ws.sorted_w,
                                    ws.rows, ws.bm, tokens, slots_bf16, status, stream)))
      return r;
  }
  if (out_bf16 && (r = b200moe_reduce_slots(slots_bf16, nullptr, tokens, out_bf16, stream))) return r;
  return 0;
}

// Block height 128: GEMM1 gathers its token rows from the row-major quantised tokens (ws.q4, ws.s4) by the sorted list, so
// no sorted copy of the activations is written (measured against gather + GEMM1: 20 to 30 us less from 1024 to 16384 tokens).
static int experts_gathering_and_reduce(const b200moe_weights* w, const Workspace& ws, int64_t tokens, void* slots_bf16,
                                        void* out_bf16, int32_t* status, void* stream) {
  const int ne = w->num_experts;
  int r;
  if ((r = b200moe_gemm1_swiglu_quant_gather(w->w13t, ne, ws.q4, ws.s4, tokens, 0, ws.sorted_ids, ws.block_expert, ws.num_valid,
                                             ws.rows, ws.hq, ws.sfh, status, stream)))
    return r;
  if ((r = b200moe_gemm2_weighted(w->w2t, ne, ws.hq, ws.sfh, ws.block_expert, ws.num_valid, ws.sorted_ids, ws.sorted_w,
                                  ws.rows, ws.bm, tokens, slots_bf16, status, stream)))
    return r;
  if (out_bf16 && (r = b200moe_reduce_slots(slots_bf16, nullptr, tokens, out_bf16, stream))) return r;
  return 0;
}
}  // namespace b200moe

extern "C" int b200moe_forward_x(const b200moe_weights* w, const void* x_bf16, int64_t tokens, void* workspace,
                                 size_t workspace_bytes, void* slots_bf16, void* out_bf16, int32_t* status,
                                 void* stream) {
  using namespace b200moe;
  if (!w || !x_bf16 || !workspace || !slots_bf16 || !status || !w->gate) return B200MOE_E_ARG;
  if (tokens < 1 || tokens > B200MOE_MAX_TOKENS) return B200MOE_E_ARG;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return B200MOE_E_ALIGN;
  const int ne = w->num_experts;
  Workspace ws = carve(static_cast<uint8_t*>(workspace), tokens, ne, true);
  if (workspace_bytes < ws.bytes) return B200MOE_E_ARG;
  const int splits = b200moe_router_splits(tokens);
  int r;
  if (tokens >= 128 && w->gate_split != nullptr) {
    // prefill sizes: the router GEMM on the tensor cores (three bf16 terms of the gate), the quantiser beside it
    if ((r = b200moe_router_gemm_tc(x_bf16, w->gate_split, tokens, ne, splits, ws.partials, status, stream))) return r;
    if ((r = quant_rows(x_bf16, tokens, ws.q4, ws.s4, stream))) return r;
  } else if ((r = b200moe_router_gemm_quant(x_bf16, w->gate, tokens, ne, splits, ws.partials, ws.q4, ws.s4, nullptr, nullptr,
                                            stream))) {  // one pass over x: logit partials and the MXFP4 operands, row-major
    return r;
  }
  if (tokens <= kSmallTokens && ne >= 4) {  // routing on the partials, sort and gather of the quantised rows in one launch
    if ((r = prep_small(ws.partials, ne, tokens * ne, splits, w->bias, tokens, ne, w->route_mode, w->route_scale, ws.bm, ws.w,
                        ws.ids, ws.sorted_ids, ws.sorted_w, ws.block_expert, ws.num_valid, nullptr, ws.q4, ws.s4, ws.rows,
                        ws.xq_sorted, ws.sfx, ws.done, static_cast<int>(ws.rows / ws.bm), stream)))
      return r;
    return experts_and_reduce(w, ws, tokens, slots_bf16, out_bf16, status, stream);
  }
  if ((r = b200moe_route_sort_partials(ws.partials, ne, tokens * ne, splits, w->bias, tokens, ne, w->route_mode,
                                       w->route_scale, ws.bm, ws.w, ws.ids, ws.sorted_ids, ws.sorted_w, ws.block_expert,
                                       ws.num_valid, ws.scratch, stream)))
    return r;
  if (ws.bm == 128) return experts_gathering_and_reduce(w, ws, tokens, slots_bf16, out_bf16, status, stream);
  if ((r = dispatch_rows_done(ws.q4, ws.s4, ws.sorted_ids, ws.num_valid, tokens, ws.bm, 0, ws.rows, ws.xq_sorted, ws.sfx,
                              ws.done, stream)))
    return r;
  return experts_and_reduce(w, ws, tokens, slots_bf16, out_bf16, status, stream);
}

extern "C" int b200moe_forward(const b200moe_weights* w, const void* x_bf16, const float* logits, int64_t tokens,
                               void* workspace, size_t workspace_bytes, void* slots_bf16, void* out_bf16,
                               int32_t* status, void* stream) {
  using namespace b200moe;
  if (!w || !x_bf16 || !logits || !workspace || !slots_bf16 || !status) return B200MOE_E_ARG;
  if (tokens < 1 || tokens > B200MOE_MAX_TOKENS) return B200MOE_E_ARG;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return B200MOE_E_ALIGN;
  const int ne = w->num_experts;
  Workspace ws = carve(static_cast<uint8_t*>(workspace), tokens, ne);
  if (workspace_bytes < ws.bytes) return B200MOE_E_ARG;
  int r;
  if (tokens <= kSmallTokens && ne >= 4) {  // routing, sort, quantisation and gather in one launch
    if ((r = prep_small(logits, ne, 0, 1, w->bias, tokens, ne, w->route_mode, w->route_scale, ws.bm, ws.w, ws.ids,
                        ws.sorted_ids, ws.sorted_w, ws.block_expert, ws.num_valid, x_bf16, nullptr, nullptr, ws.rows,
                        ws.xq_sorted, ws.sfx, ws.done, static_cast<int>(ws.rows / ws.bm), stream)))
      return r;
    return experts_and_reduce(w, ws, tokens, slots_bf16, out_bf16, status, stream);
  }
  if ((r = b200moe_route_sort(logits, w->bias, tokens, ne, w->route_mode, w->route_scale, ws.bm, ws.w, ws.ids,
                              ws.sorted_ids, ws.sorted_w, ws.block_expert, ws.num_valid, ws.scratch, stream)))
    return r;
  if (ws.bm == 128) {
    // prefill sizes: quantise every token once (row-major); GEMM1 gathers the rows itself
    if ((r = quant_rows(x_bf16, tokens, ws.q4, ws.s4, stream))) return r;
    return experts_gathering_and_reduce(w, ws, tokens, slots_bf16, out_bf16, status, stream);
  } else if ((r = b200moe_quant_dispatch(x_bf16, ws.sorted_ids, ws.num_valid, tokens, ws.bm, ws.rows, ws.xq_sorted, ws.sfx,
                                         ws.done, stream))) {
    return r;
  }
  return experts_and_reduce(w, ws, tokens, slots_bf16, out_bf16, status, stream);
}

extern "C" int b200moe_forward_host(const b200moe_weights* w, const void* host_x_bf16, const float* host_logits,
                                    int64_t tokens, void* dev_x, float* dev_logits, void* workspace,
                                    size_t workspace_bytes, void* slots_bf16, void* dev_out, void* host_out_bf16,
                                    int32_t* status, void* stream) {
  using namespace b200moe;
  if (!w || !host_x_bf16 || !host_logits || !dev_x || !dev_logits || !dev_out || !host_out_bf16) return B200MOE_E_ARG;
  if (tokens < 1 || tokens > B200MOE_MAX_TOKENS) return B200MOE_E_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(dev_x, host_x_bf16, tokens * kH * 2, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemcpyAsync(dev_logits, host_logits, tokens * w->num_experts * 4, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int r = b200moe_forward(w, dev_x, dev_logits, tokens, workspace, workspace_bytes, slots_bf16, dev_out, status, stream);
  if (r) return r;
  e = cudaMemcpyAsync(host_out_bf16, dev_out, tokens * kH * 2, cudaMemcpyDeviceToHost, s);
  return e == cudaSuccess ? 0 : static_cast<int>(e);
}
