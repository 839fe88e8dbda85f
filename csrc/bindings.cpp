// Python bindings: torch tensors -> the C ABI in api.h.  Also hosts the small C++ runtime pieces
// (weak_ref_tensor, tensor-map cache, GEMM workspace).
//
// weak_ref_tensor mirrors the one native function of the reference (vllm_kunlun/csrc/utils.cpp:4-32):
// an alias of a CUDA tensor that does not own its storage, used to hold CUDA-graph outputs without
// keeping the allocation alive.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

#include "api.h"

namespace {

int dtype_code(const at::Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return 0;
    case at::kBFloat16: return 1;
    case at::kHalf: return 2;
    default: TORCH_CHECK(false, "unsupported dtype ", t.scalar_type());
  }
}
cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }
std::atomic<int64_t> g_launches{0};
void check(int rc, const char* what, int n_kernels = 1) {
  TORCH_CHECK(rc == 0, what, " failed with code ", rc);
  g_launches += n_kernels;
}
int64_t launch_count() { return g_launches.load(); }
const void* opt_ptr(const c10::optional<at::Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }

at::Tensor weak_ref_tensor(const at::Tensor& t) {
  TORCH_CHECK(t.is_cuda(), "weak_ref_tensor expects a CUDA tensor");
  return torch::from_blob(t.data_ptr(), t.sizes(), t.strides(), t.options());
}

}  // namespace

// Dispatcher registration (the reference registers the same function as ``torch.ops._C.weak_ref_tensor``,
// vllm_kunlun/csrc/utils.cpp:26-28).  The op lives in this library's own namespace because an installed vLLM
// defines ``_C::weak_ref_tensor`` itself and a second definition would abort the load; the Python loader aliases it
// into ``_C`` when that name is still free.
TORCH_LIBRARY(_C_b200, m) { m.def("weak_ref_tensor(Tensor input) -> Tensor"); }
TORCH_LIBRARY_IMPL(_C_b200, CUDA, m) { m.impl("weak_ref_tensor", &weak_ref_tensor); }

namespace {

// ---------------------------------------------------------------------------------------- GEMM
struct TmapKey {
  const void* p; int64_t rows, cols, stride; int box_rows; int elem_bytes;
  bool operator==(const TmapKey& o) const {
    return p == o.p && rows == o.rows && cols == o.cols && stride == o.stride && box_rows == o.box_rows &&
           elem_bytes == o.elem_bytes;
  }
};
struct TmapHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = std::hash<const void*>()(k.p);
    h ^= std::hash<int64_t>()(k.rows * 1315423911u + k.cols) + 0x9e3779b9 + (h << 6) + (h >> 2);
    h ^= std::hash<int64_t>()((k.stride * 31 + k.box_rows) * 4 + k.elem_bytes) + 0x9e3779b9 + (h << 6) + (h >> 2);
    return h;
  }
};
struct alignas(64) Tmap { unsigned char b[128]; };

struct GemmState {
  std::mutex mu;
  std::unordered_map<TmapKey, Tmap, TmapHash> cache;
  at::Tensor ws, counters, status;
  int num_sms = 0;
  int64_t launches = 0;
};
GemmState& gemm_state() { static GemmState s; return s; }

const Tmap& get_tmap(GemmState& gs, const at::Tensor& t, int box_rows, int elem_bytes) {
  TmapKey key{t.data_ptr(), t.size(0), t.size(1), t.stride(0), box_rows, elem_bytes};
  auto it = gs.cache.find(key);
  if (it != gs.cache.end()) return it->second;
  if (gs.cache.size() > 4096) gs.cache.clear();
  Tmap tm;
  int rc = b200_encode_tmap_2d(tm.b, t.data_ptr(), t.size(0), t.size(1), t.stride(0) * elem_bytes, box_rows,
                               128 / elem_bytes, elem_bytes);
  TORCH_CHECK(rc == 0, "tensor map encode failed: ", rc);
  return gs.cache.emplace(key, tm).first->second;
}

// Plain (unswizzled) byte tensor map with a [box_rows, box_bytes] box; cached under elem_bytes = -box_bytes.
const Tmap& get_tmap_raw(GemmState& gs, const at::Tensor& t, int box_rows, int box_bytes) {
  TmapKey key{t.data_ptr(), t.size(0), t.size(1), t.stride(0), box_rows, -box_bytes};
  auto it = gs.cache.find(key);
  if (it != gs.cache.end()) return it->second;
  if (gs.cache.size() > 4096) gs.cache.clear();
  Tmap tm;
  int rc = b200_encode_tmap_2d_raw(tm.b, t.data_ptr(), t.size(0), t.size(1), t.stride(0), box_rows, box_bytes);
  TORCH_CHECK(rc == 0, "tensor map encode failed: ", rc);
  return gs.cache.emplace(key, tm).first->second;
}

// Collective-fusion arguments for the NEXT gemm() call (consumed by it).
struct GemmCommState {
  bool active = false;
  void* rs_stage[8] = {nullptr}; void* rs_flags[8] = {nullptr}; const void* ag_flags = nullptr;
  int rs_on = 0, rs_tloc = 0, rs_rank = 0, ag_on = 0, ag_expect = 0;
};
GemmCommState g_comm;
void set_gemm_comm(std::vector<int64_t> rs_stage, std::vector<int64_t> rs_flags, int64_t ag_flags, int64_t rs_tloc,
                   int64_t rs_rank, int64_t ag_expect) {
  g_comm = GemmCommState();
  g_comm.active = true;
  for (size_t i = 0; i < rs_stage.size() && i < 8; ++i) {
    g_comm.rs_stage[i] = reinterpret_cast<void*>(rs_stage[i]);
    g_comm.rs_flags[i] = reinterpret_cast<void*>(rs_flags[i]);
  }
  g_comm.rs_on = rs_stage.empty() ? 0 : 1;
  g_comm.rs_tloc = rs_tloc; g_comm.rs_rank = rs_rank;
  g_comm.ag_flags = reinterpret_cast<const void*>(ag_flags);
  g_comm.ag_on = ag_flags != 0;
  g_comm.ag_expect = ag_expect;
}

// out[T, N] = x[T, K] @ w[N, K]^T (+ bias).  splits <= 0 lets the library choose.
void gemm(at::Tensor out, const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& bias,
          int64_t splits, int64_t bn_override, int64_t stages, int64_t ctas_per_sm, int64_t act) {
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && out.is_cuda());
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2);
  TORCH_CHECK(x.scalar_type() == w.scalar_type() && x.scalar_type() == out.scalar_type());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf, "gemm: bf16/fp16 only");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && out.stride(1) == 1);
  const int T = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K && out.size(0) == T && out.size(1) == (act ? N / 2 : N));
  if (act) {
    TORCH_CHECK(N % 128 == 0 && out.stride(0) % 8 == 0, "fused gate/up activation needs whole [64 | 64] weight tiles");
    splits = 1;  // whole tiles only: both halves of a feature pair must meet in one epilogue
  }
  TORCH_CHECK(K % 8 == 0 && x.stride(0) % 8 == 0 && w.stride(0) % 8 == 0, "gemm: K and row strides must be multiples of 8");
  if (T == 0 || N == 0) return;
  c10::cuda::CUDAGuard guard(x.device());
  GemmState& gs = gemm_state();
  std::lock_guard<std::mutex> lk(gs.mu);
  if (gs.num_sms == 0) {
    gs.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    gs.ws = at::empty({16 << 20}, x.options().dtype(at::kFloat));        // 64 MiB of split-K partials
    gs.counters = at::zeros({1 << 16}, x.options().dtype(at::kInt));
    gs.status = at::zeros({1}, x.options().dtype(at::kInt));
  }
  GemmArgs a;
  memset(&a, 0, sizeof(a));
  a.spin_limit = 1u << 22;
  if (g_comm.active) {  // one-shot: collective fusion requested for this launch (set_gemm_comm)
    for (int i = 0; i < 8; ++i) { a.rs_stage[i] = g_comm.rs_stage[i]; a.rs_flags[i] = g_comm.rs_flags[i]; }
    a.ag_flags = g_comm.ag_flags; a.rs_on = g_comm.rs_on; a.rs_tloc = g_comm.rs_tloc; a.rs_rank = g_comm.rs_rank;
    a.ag_on = g_comm.ag_on; a.ag_expect = g_comm.ag_expect;
    g_comm.active = false;
  }
  a.bn = bn_override > 0 ? (int)bn_override : b200_gemm_pick_bn(T);
  a.T = T; a.N = N; a.K = K;
  a.n_tiles = (N + 127) / 128;
  a.t_tiles = (T + a.bn - 1) / a.bn;
  const int total_kb = (K + 63) / 64;
  const int tiles = a.n_tiles * a.t_tiles;
  const int cps = ctas_per_sm > 0 ? (int)ctas_per_sm : 1;
  const int slots = gs.num_sms * cps;
  const int64_t units = (int64_t)tiles * total_kb;
  // splits == 1 forces whole tiles; splits > 1 forces ceil(total_kb / splits) units per CTA;
  // otherwise whole tiles when there are many of them per SM, stream-K when there are few.
  int per = 0;
  if (splits > 1) {
    per = (total_kb + (int)splits - 1) / (int)splits;
  } else if (splits <= 0) {
    // Whole tiles cost nothing extra; stream-K pays a fix-up (partials through L2 + an atomic
    // ticket, a few microseconds) and wins only when whole tiles would leave most SMs idle or
    // make the slowest SM stream at least twice its fair share of the weights.
    int64_t fair = std::max<int64_t>(4, (units + slots - 1) / slots);
    int64_t whole_path = (int64_t)((tiles + slots - 1) / slots) * total_kb;
    if (tiles < slots / 4 || whole_path >= 2 * fair) per = (int)fair;
    if (tiles >= 2 * slots) per = 0;
    if (a.t_tiles == 1 && !a.rs_on && !a.ag_on) {
      // Decode-shaped calls: split every tile's K range into 2 (or, for long K, 4) EQUAL parts, as long as all parts
      // fit the SMs in one round.  Measured over the decode shapes of an 8B model at TP 1-8, aligned halves /
      // quarters beat the fair-share stream-K split (fewer contributors per tile, no ranges straddling two tiles:
      // 16x768x4096 22.5 -> 16.3 us, 16x4096x4096 20.5 -> 18.4 us, 16x4096x14336 32.8 -> 31.5 us) and whole tiles.
      int k = 1;
      if (tiles * 4 <= gs.num_sms && total_kb >= 96) k = 4;
      else if (tiles * 2 <= gs.num_sms && total_kb >= 16) k = 2;
      per = k > 1 ? (total_kb + k - 1) / k : 0;
    }
  }
  if (per > 0) {
    int max_contrib = (total_kb + per - 1) / per + 1;
    int64_t grid = (units + per - 1) / per;
    if ((int64_t)tiles * max_contrib * a.bn * 128 > gs.ws.numel() || tiles > gs.counters.numel()) per = 0;
    else { a.per_cta = per; a.max_contrib = max_contrib; a.grid = (int)grid; }
  }
  if (per == 0) { a.per_cta = 0; a.max_contrib = 1; a.grid = std::min(tiles, slots); }
  a.out = out.data_ptr();
  a.bias = opt_ptr(bias);
  a.ws = gs.ws.data_ptr<float>();
  a.counters = gs.counters.data_ptr<int>();
  a.status = gs.status.data_ptr<int>();
  a.fmt = x.scalar_type() == at::kBFloat16 ? 1 : 0;
  a.ldo = out.stride(0);
  a.num_sms = gs.num_sms;
  a.stages = (int)stages;
  a.ctas_per_sm = (int)ctas_per_sm;
  a.act = (int)act;
  const Tmap& tw = get_tmap(gs, w, 128, 2);
  const Tmap& tx = get_tmap(gs, x, a.bn, 2);
  check(b200_gemm_launch(&a, tw.b, tx.b, stream()), "gemm launch");
  gs.launches++;
}

// (q int8 [rows, K], scale float [rows]); static_scale: a one-element tensor for per-tensor static quantisation.
std::vector<at::Tensor> quant_int8_token(const at::Tensor& x, const c10::optional<at::Tensor>& static_scale) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.is_cuda());
  if (static_scale.has_value()) TORCH_CHECK(static_scale->scalar_type() == at::kFloat && static_scale->numel() >= 1);
  auto q = at::empty({x.size(0), x.size(1)}, x.options().dtype(at::kChar));
  auto s = at::empty({x.size(0)}, x.options().dtype(at::kFloat));
  check(b200_quant_int8_token(q.data_ptr(), s.data_ptr<float>(), x.data_ptr(),
                              static_scale.has_value() ? static_scale->data_ptr<float>() : nullptr, x.size(0),
                              (int)x.size(1), x.stride(0), dtype_code(x), stream()),
        "quant_int8_token");
  return {q, s};
}

// W8A8 int8 linear on kind::i8: out[T, N] = (xq[T, K] . w[N, K]^T) * a_scale[T] * w_scale[N] (+ bias); s32 accumulation.
// At most 32 rows go to the cluster split-K kernel, larger batches to the dense kernel in whole tiles.
void gemm_int8(at::Tensor out, const at::Tensor& xq, const at::Tensor& w, const c10::optional<at::Tensor>& bias,
               const at::Tensor& a_scale, const at::Tensor& w_scale) {
  TORCH_CHECK(xq.is_cuda() && w.is_cuda() && out.is_cuda() && xq.dim() == 2 && w.dim() == 2 && out.dim() == 2);
  TORCH_CHECK(xq.scalar_type() == at::kChar && w.scalar_type() == at::kChar, "gemm_int8: int8 operands");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 || out.scalar_type() == at::kHalf);
  TORCH_CHECK(xq.stride(1) == 1 && w.stride(1) == 1 && out.stride(1) == 1);
  const int T = xq.size(0), K = xq.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K && out.size(0) == T && out.size(1) == N);
  TORCH_CHECK(K % 16 == 0 && xq.stride(0) % 16 == 0 && w.stride(0) % 16 == 0, "gemm_int8: K and row strides: multiples of 16");
  TORCH_CHECK(a_scale.scalar_type() == at::kFloat && a_scale.is_contiguous() && a_scale.numel() >= T);
  TORCH_CHECK(w_scale.scalar_type() == at::kFloat && w_scale.is_contiguous() && w_scale.numel() == N);
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == out.scalar_type() && bias->numel() == N);
  if (T == 0 || N == 0) return;
  c10::cuda::CUDAGuard guard(xq.device());
  GemmState& gs = gemm_state();
  std::lock_guard<std::mutex> lk(gs.mu);
  if (gs.num_sms == 0) {
    gs.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    gs.ws = at::empty({16 << 20}, out.options().dtype(at::kFloat));
    gs.counters = at::zeros({1 << 16}, out.options().dtype(at::kInt));
    gs.status = at::zeros({1}, out.options().dtype(at::kInt));
  }
  const int total_kb = (K + 127) / 128;
  const int fmt = out.scalar_type() == at::kBFloat16 ? 1 : 0;
  if (T <= 32) {
    GemmDecodeArgs a;
    memset(&a, 0, sizeof(a));
    a.out = out.data_ptr(); a.bias = opt_ptr(bias); a.status = gs.status.data_ptr<int>();
    a.T = T; a.N = N; a.K = K;
    a.n_tiles = (N + 127) / 128;
    a.bn = T <= 16 ? 16 : 32;
    a.fmt = fmt; a.ldo = out.stride(0);
    a.i8 = 1; a.a_scale = a_scale.data_ptr<float>(); a.w_scale = w_scale.data_ptr<float>();
    const int max_s = a.bn == 16 ? 8 : 4;
    int S = 1;
    while (S * 2 <= max_s && a.n_tiles * S * 2 <= gs.num_sms && total_kb / (S * 2) >= 4) S *= 2;
    while (S > 1 && (S - 1) * ((total_kb + S - 1) / S) >= total_kb) --S;
    a.S = S;
    a.kb_per_cta = (total_kb + S - 1) / S;
    a.ctas_per_sm = a.n_tiles * S > gs.num_sms ? 2 : 1;
    const Tmap& tw = get_tmap(gs, w, 128, 1);
    const Tmap& tx = get_tmap(gs, xq, a.bn, 1);
    check(b200_gemm_decode_launch(&a, tw.b, tx.b, stream()), "gemm_int8 (decode) launch");
  } else {
    GemmArgs a;
    memset(&a, 0, sizeof(a));
    a.spin_limit = 1u << 22;
    a.bn = b200_gemm_pick_bn(T);
    a.T = T; a.N = N; a.K = K;
    a.n_tiles = (N + 127) / 128;
    a.t_tiles = (T + a.bn - 1) / a.bn;
    a.per_cta = 0; a.max_contrib = 1;
    a.grid = std::min(a.n_tiles * a.t_tiles, gs.num_sms);
    a.out = out.data_ptr(); a.bias = opt_ptr(bias); a.ws = gs.ws.data_ptr<float>();
    a.counters = gs.counters.data_ptr<int>(); a.status = gs.status.data_ptr<int>();
    a.fmt = fmt; a.ldo = out.stride(0); a.num_sms = gs.num_sms;
    a.i8 = 1; a.a_scale = a_scale.data_ptr<float>(); a.w_scale = w_scale.data_ptr<float>();
    const Tmap& tw = get_tmap(gs, w, 128, 1);
    const Tmap& tx = get_tmap(gs, xq, a.bn, 1);
    check(b200_gemm_launch(&a, tw.b, tx.b, stream()), "gemm_int8 launch");
  }
  gs.launches++;
}

// Row-parallel push epilogue for the NEXT gemm_decode() call: the output is also written, as {data, epoch} units,
// into the low-latency all-reduce slots of every peer (consumed by ll_allreduce(..., skip_push = true)).
struct DecCommState {
  bool active = false;
  void* ll_bufs[8] = {nullptr};
  const void* epoch_word = nullptr;
  int64_t slot_bytes = 0;
  int rank = 0, nranks = 0;
};
DecCommState g_dec_comm;
void set_gemm_decode_comm(std::vector<int64_t> ll_bufs, at::Tensor epochs, int64_t slot_bytes, int64_t rank) {
  g_dec_comm = DecCommState();
  TORCH_CHECK(ll_bufs.size() <= 8 && ll_bufs.size() >= 2);
  g_dec_comm.active = true;
  for (size_t i = 0; i < ll_bufs.size(); ++i) g_dec_comm.ll_bufs[i] = reinterpret_cast<void*>(ll_bufs[i]);
  g_dec_comm.epoch_word = epochs.data_ptr<int>();
  g_dec_comm.slot_bytes = slot_bytes;
  g_dec_comm.rank = rank;
  g_dec_comm.nranks = ll_bufs.size();
}

// Decode-sized GEMM (T <= 32): cluster split-K with the reduction in distributed shared memory.
// splits <= 0 lets the library choose the cluster size.
void gemm_decode(at::Tensor out, const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& bias,
                 int64_t splits, int64_t stages, int64_t ctas_per_sm, int64_t act) {
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && out.is_cuda());
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && out.dim() == 2);
  TORCH_CHECK(x.scalar_type() == w.scalar_type() && x.scalar_type() == out.scalar_type());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf, "gemm_decode: bf16/fp16 only");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && out.stride(1) == 1);
  const int T = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(T <= 32, "gemm_decode: at most 32 rows");
  TORCH_CHECK(w.size(1) == K && out.size(0) == T && out.size(1) == (act ? N / 2 : N));
  if (act) TORCH_CHECK(N % 128 == 0 && out.stride(0) % 8 == 0, "fused gate/up activation needs whole [64 | 64] weight tiles");
  TORCH_CHECK(K % 8 == 0 && x.stride(0) % 8 == 0 && w.stride(0) % 8 == 0, "gemm_decode: K and row strides must be multiples of 8");
  if (T == 0 || N == 0) return;
  c10::cuda::CUDAGuard guard(x.device());
  GemmState& gs = gemm_state();
  std::lock_guard<std::mutex> lk(gs.mu);
  if (gs.num_sms == 0) {
    gs.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    gs.ws = at::empty({16 << 20}, x.options().dtype(at::kFloat));
    gs.counters = at::zeros({1 << 16}, x.options().dtype(at::kInt));
    gs.status = at::zeros({1}, x.options().dtype(at::kInt));
  }
  GemmDecodeArgs a;
  memset(&a, 0, sizeof(a));
  a.out = out.data_ptr(); a.bias = opt_ptr(bias); a.status = gs.status.data_ptr<int>();
  a.T = T; a.N = N; a.K = K;
  a.n_tiles = (N + 127) / 128;
  a.bn = T <= 16 ? 16 : 32;
  a.fmt = x.scalar_type() == at::kBFloat16 ? 1 : 0;
  a.ldo = out.stride(0);
  a.act = (int)act;
  const int total_kb = (K + 63) / 64;
  const int max_s = a.bn == 16 ? 8 : 4;
  int S = (int)splits;
  if (S <= 0) {
    // Measured in graph chains over the decode shapes of an 8B model at TP 1-8 (benchmarks/bench_gemm_decode_sweep.py):
    // the largest power-of-two cluster that keeps all CTAs on distinct SMs and leaves every CTA at least 8 k-blocks
    // (128 KB of weights) wins or ties; odd cluster sizes schedule badly; a cluster costs about 1 us over S = 1.
    S = 1;
    while (S * 2 <= max_s && a.n_tiles * S * 2 <= gs.num_sms && total_kb / (S * 2) >= 8) S *= 2;
  }
  S = std::max(1, std::min(S, std::min(max_s, total_kb)));
  while (S > 1 && (S - 1) * ((total_kb + S - 1) / S) >= total_kb) --S;  // no CTA without work
  a.S = S;
  a.kb_per_cta = (total_kb + S - 1) / S;
  a.stages = (int)stages;
  a.ctas_per_sm = ctas_per_sm > 0 ? (int)ctas_per_sm : (a.n_tiles * S > gs.num_sms ? 2 : 1);
  if (g_dec_comm.active) {
    TORCH_CHECK(!act && N % 8 == 0 && out.stride(0) == N, "push epilogue needs a contiguous [T, N] output");
    TORCH_CHECK((int64_t)T * N * 4 <= g_dec_comm.slot_bytes, "push epilogue: payload exceeds the all-reduce slot");
    a.ar_on = 1; a.rank = g_dec_comm.rank; a.nranks = g_dec_comm.nranks;
    for (int i = 0; i < 8; ++i) a.ll_bufs[i] = g_dec_comm.ll_bufs[i];
    a.epoch_word = g_dec_comm.epoch_word; a.ll_slot_bytes = g_dec_comm.slot_bytes;
    g_dec_comm.active = false;
  }
  const Tmap& tw = get_tmap(gs, w, 128, 2);
  const Tmap& tx = get_tmap(gs, x, a.bn, 2);
  check(b200_gemm_decode_launch(&a, tw.b, tx.b, stream()), "gemm_decode launch");
  gs.launches++;
}

// Decode-sized linear over 4-bit weights (AWQ / GPTQ after repacking, see quantization/int4.py::pack_w4):
// out [T <= 32, N] = x [T, K] . W^T with W[n, k] = (q[n, k] - zero[n, k / group]) * scale[n, k / group], the packed bytes
// streamed from HBM and de-quantised inside the kernel.  act as in gemm_decode (interleaved gate / up rows).
void gemm_decode_w4(at::Tensor out, const at::Tensor& x, const at::Tensor& packed, const at::Tensor& scale, const at::Tensor& zero,
                    const c10::optional<at::Tensor>& bias, int64_t group, int64_t splits, int64_t act) {
  TORCH_CHECK(x.is_cuda() && packed.is_cuda() && out.is_cuda() && x.dim() == 2 && packed.dim() == 2 && out.dim() == 2);
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf, "gemm_decode_w4: bf16/fp16 activations");
  TORCH_CHECK(packed.scalar_type() == at::kByte && packed.is_contiguous() && x.stride(1) == 1 && out.stride(1) == 1);
  TORCH_CHECK(scale.scalar_type() == x.scalar_type() && zero.scalar_type() == x.scalar_type() && out.scalar_type() == x.scalar_type());
  const int T = x.size(0), K = x.size(1), N = packed.size(0);
  TORCH_CHECK(T <= 32, "gemm_decode_w4: at most 32 rows");
  TORCH_CHECK(packed.size(1) * 2 == K && out.size(0) == T && out.size(1) == (act ? N / 2 : N));
  TORCH_CHECK(K % 64 == 0 && group >= 64 && group % 64 == 0 && K % group == 0 && x.stride(0) % 8 == 0,
              "gemm_decode_w4: K and the group size must be multiples of 64");
  TORCH_CHECK(scale.is_contiguous() && zero.is_contiguous() && scale.dim() == 2 && scale.size(0) == N &&
              scale.size(1) == K / group && zero.sizes() == scale.sizes());
  if (act) TORCH_CHECK(N % 128 == 0 && out.stride(0) % 8 == 0, "fused gate/up activation needs whole [64 | 64] weight tiles");
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == out.scalar_type() && bias->numel() == N);
  if (T == 0 || N == 0) return;
  c10::cuda::CUDAGuard guard(x.device());
  GemmState& gs = gemm_state();
  std::lock_guard<std::mutex> lk(gs.mu);
  if (gs.num_sms == 0) {
    gs.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    gs.ws = at::empty({16 << 20}, x.options().dtype(at::kFloat));
    gs.counters = at::zeros({1 << 16}, x.options().dtype(at::kInt));
    gs.status = at::zeros({1}, x.options().dtype(at::kInt));
  }
  GemmDecodeArgs a;
  memset(&a, 0, sizeof(a));
  a.out = out.data_ptr(); a.bias = opt_ptr(bias); a.status = gs.status.data_ptr<int>();
  a.T = T; a.N = N; a.K = K;
  a.n_tiles = (N + 127) / 128;
  a.bn = T <= 16 ? 16 : 32;
  a.fmt = x.scalar_type() == at::kBFloat16 ? 1 : 0;
  a.ldo = out.stride(0);
  a.act = (int)act;
  a.w4 = 1; a.w4_group = (int)group; a.w4_scale = scale.data_ptr(); a.w4_zero = zero.data_ptr();
  const int total_kb = K / 64;
  const int max_s = a.bn == 16 ? 8 : 4;
  int S = (int)splits;
  if (S <= 0) {
    // the de-quantising warps of a CTA bound its throughput, so more CTAs help where 16-bit weights would already be
    // bandwidth-bound: clusters of up to 4 may fill the SMs twice (two CTAs fit per SM), larger ones once
    S = 1;
    while (S * 2 <= max_s && total_kb / (S * 2) >= 8 && a.n_tiles * S * 2 <= (S * 2 <= 4 ? 2 : 1) * gs.num_sms) S *= 2;
  }
  S = std::max(1, std::min(S, std::min(max_s, total_kb)));
  while (S > 1 && (S - 1) * ((total_kb + S - 1) / S) >= total_kb) --S;
  a.S = S;
  a.kb_per_cta = (total_kb + S - 1) / S;
  a.ctas_per_sm = a.n_tiles * S > gs.num_sms ? 2 : 1;
  const Tmap& tw = get_tmap_raw(gs, packed, 128, 32);
  const Tmap& tx = get_tmap(gs, x, a.bn, 2);
  check(b200_gemm_decode_launch(&a, tw.b, tx.b, stream()), "gemm_decode_w4 launch");
  gs.launches++;
}

// 4-bit weights -> a 16-bit [N, K] matrix (for batches the decode kernel does not take).
void dequant_w4(at::Tensor out, const at::Tensor& packed, const at::Tensor& scale, const at::Tensor& zero, int64_t group) {
  TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.dim() == 2 && packed.is_contiguous() && packed.scalar_type() == at::kByte);
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 || out.scalar_type() == at::kHalf);
  TORCH_CHECK(scale.scalar_type() == out.scalar_type() && zero.scalar_type() == out.scalar_type());
  const int64_t N = out.size(0);
  const int K = out.size(1);
  TORCH_CHECK(packed.size(0) == N && packed.size(1) * 2 == K && scale.is_contiguous() && zero.is_contiguous());
  TORCH_CHECK(K % group == 0 && scale.numel() == N * (K / group) && zero.numel() == scale.numel());
  c10::cuda::CUDAGuard guard(out.device());
  check(b200_dequant_w4(out.data_ptr(), packed.data_ptr(), scale.data_ptr(), zero.data_ptr(), N, K, (int)group,
                        dtype_code(out), stream()), "dequant_w4");
}

// qkv projection of a decode-sized batch with split + optional q / k RMSNorm + rotary + K / V cache write in the GEMM
// epilogue (head_dim 128, full rotary dim).  q_out [T, Hq * 128]; w [(Hq + 2 Hkv) * 128, K].
void gemm_decode_qkv(at::Tensor q_out, const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& bias,
                     const at::Tensor& positions, const at::Tensor& cos_sin, const c10::optional<at::Tensor>& q_w,
                     const c10::optional<at::Tensor>& k_w, double eps, int64_t Hq, int64_t Hkv, bool neox, bool gemma,
                     const c10::optional<at::Tensor>& kv_cache, const at::Tensor& slots) {
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && q_out.is_cuda() && x.dim() == 2 && w.dim() == 2 && q_out.dim() == 2);
  TORCH_CHECK(x.scalar_type() == w.scalar_type() && x.scalar_type() == q_out.scalar_type());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf, "gemm_decode_qkv: bf16/fp16 only");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && q_out.is_contiguous());
  const int T = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(T <= 32 && w.size(1) == K && N == (Hq + 2 * Hkv) * 128 && q_out.size(0) == T && q_out.size(1) == Hq * 128);
  TORCH_CHECK(K % 8 == 0 && x.stride(0) % 8 == 0 && w.stride(0) % 8 == 0);
  TORCH_CHECK(positions.scalar_type() == at::kLong && positions.is_contiguous() && positions.numel() >= T);
  TORCH_CHECK(slots.scalar_type() == at::kLong && slots.is_contiguous() && slots.numel() >= T);
  TORCH_CHECK(cos_sin.scalar_type() == at::kFloat && cos_sin.is_contiguous() && cos_sin.size(-1) == 128,
              "gemm_decode_qkv: rotary dim 128");
  if (q_w.has_value()) TORCH_CHECK(q_w->scalar_type() == x.scalar_type() && q_w->numel() == 128 && q_w->is_contiguous());
  if (k_w.has_value()) TORCH_CHECK(k_w->scalar_type() == x.scalar_type() && k_w->numel() == 128 && k_w->is_contiguous());
  if (kv_cache.has_value())
    TORCH_CHECK(kv_cache->is_contiguous() && kv_cache->scalar_type() == x.scalar_type() && kv_cache->dim() == 5 &&
                kv_cache->size(1) == 2 && kv_cache->size(2) == Hkv && kv_cache->size(4) == 128);
  if (T == 0) return;
  c10::cuda::CUDAGuard guard(x.device());
  GemmState& gs = gemm_state();
  std::lock_guard<std::mutex> lk(gs.mu);
  if (gs.num_sms == 0) {
    gs.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    gs.ws = at::empty({16 << 20}, x.options().dtype(at::kFloat));
    gs.counters = at::zeros({1 << 16}, x.options().dtype(at::kInt));
    gs.status = at::zeros({1}, x.options().dtype(at::kInt));
  }
  GemmDecodeArgs a;
  memset(&a, 0, sizeof(a));
  a.out = q_out.data_ptr(); a.bias = opt_ptr(bias); a.status = gs.status.data_ptr<int>();
  a.T = T; a.N = N; a.K = K;
  a.n_tiles = N / 128;
  a.bn = T <= 16 ? 16 : 32;
  a.fmt = x.scalar_type() == at::kBFloat16 ? 1 : 0;
  a.ldo = q_out.stride(0);
  const int total_kb = (K + 63) / 64;
  const int max_s = a.bn == 16 ? 8 : 4;
  int S = 1;
  while (S * 2 <= max_s && a.n_tiles * S * 2 <= gs.num_sms && total_kb / (S * 2) >= 8) S *= 2;
  while (S > 1 && (S - 1) * ((total_kb + S - 1) / S) >= total_kb) --S;
  a.S = S;
  a.kb_per_cta = (total_kb + S - 1) / S;
  a.ctas_per_sm = a.n_tiles * S > gs.num_sms ? 2 : 1;
  a.qk_on = 1; a.qk_hq = (int)Hq; a.qk_hkv = (int)Hkv; a.qk_neox = neox; a.qk_gemma = gemma; a.qk_eps = (float)eps;
  a.qk_positions = positions.data_ptr<int64_t>(); a.qk_cos_sin = cos_sin.data_ptr<float>();
  a.qk_q_w = q_w.has_value() ? q_w->data_ptr() : nullptr;
  a.qk_k_w = k_w.has_value() ? k_w->data_ptr() : nullptr;
  a.qk_kv_cache = kv_cache.has_value() ? kv_cache->data_ptr() : nullptr;
  a.qk_slots = slots.data_ptr<int64_t>();
  a.qk_block_size = kv_cache.has_value() ? (int)kv_cache->size(3) : 1;
  a.qk_num_blocks = kv_cache.has_value() ? kv_cache->size(0) : 0;
  a.qk_max_pos = cos_sin.size(0);
  const Tmap& tw = get_tmap(gs, w, 128, 2);
  const Tmap& tx = get_tmap(gs, x, a.bn, 2);
  check(b200_gemm_decode_launch(&a, tw.b, tx.b, stream()), "gemm_decode_qkv launch");
  gs.launches++;
}

// fp8 block-scaled decode GEMM (T <= 32): xq [T, K] e4m3 with transposed 1x128 scales a_scale_t [K/128, stride],
// w [N, K] e4m3 with w_scale [ceil(N/128), ceil(K/128)]; cluster split-K like gemm_decode.
void gemm_decode_fp8(at::Tensor out, const at::Tensor& xq, const at::Tensor& w, const c10::optional<at::Tensor>& bias,
                     const at::Tensor& a_scale_t, const at::Tensor& w_scale, int64_t splits) {
  TORCH_CHECK(xq.is_cuda() && w.is_cuda() && out.is_cuda() && xq.dim() == 2 && w.dim() == 2 && out.dim() == 2);
  TORCH_CHECK(xq.element_size() == 1 && w.element_size() == 1, "gemm_decode_fp8: 8-bit operands");
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 || out.scalar_type() == at::kHalf);
  TORCH_CHECK(xq.stride(1) == 1 && w.is_contiguous() && out.stride(1) == 1);
  const int T = xq.size(0), K = xq.size(1), N = w.size(0);
  TORCH_CHECK(T <= 32 && w.size(1) == K && out.size(0) == T && out.size(1) == N);
  TORCH_CHECK(K % 16 == 0 && xq.stride(0) % 16 == 0, "gemm_decode_fp8: K and the row stride must be multiples of 16");
  const int total_kb = (K + 127) / 128;
  TORCH_CHECK(a_scale_t.scalar_type() == at::kFloat && a_scale_t.dim() == 2 && a_scale_t.stride(1) == 1 &&
              a_scale_t.size(0) >= total_kb && a_scale_t.size(1) >= T);
  TORCH_CHECK(w_scale.scalar_type() == at::kFloat && w_scale.is_contiguous() && w_scale.numel() == (int64_t)((N + 127) / 128) * total_kb);
  if (T == 0 || N == 0) return;
  c10::cuda::CUDAGuard guard(xq.device());
  GemmState& gs = gemm_state();
  std::lock_guard<std::mutex> lk(gs.mu);
  if (gs.num_sms == 0) {
    gs.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    gs.ws = at::empty({16 << 20}, out.options().dtype(at::kFloat));
    gs.counters = at::zeros({1 << 16}, out.options().dtype(at::kInt));
    gs.status = at::zeros({1}, out.options().dtype(at::kInt));
  }
  GemmDecodeArgs a;
  memset(&a, 0, sizeof(a));
  a.out = out.data_ptr(); a.bias = opt_ptr(bias); a.status = gs.status.data_ptr<int>();
  a.T = T; a.N = N; a.K = K;
  a.n_tiles = (N + 127) / 128;
  a.bn = T <= 16 ? 16 : 32;
  a.fmt = out.scalar_type() == at::kBFloat16 ? 1 : 0;
  a.ldo = out.stride(0);
  a.fp8 = 1; a.a_scale = a_scale_t.data_ptr<float>(); a.w_scale = w_scale.data_ptr<float>(); a.a_stride = a_scale_t.stride(0);
  const int max_s = a.bn == 16 ? 8 : 4;
  int S = (int)splits;
  if (S <= 0) {
    // measured: a cluster of 8 only pays when each CTA still has >= 7 k-blocks (16 KB of weights each); below that
    // the 7-way partial exchange costs more than the extra SMs bring
    S = 1;
    while (S * 2 <= max_s && a.n_tiles * S * 2 <= gs.num_sms && total_kb / (S * 2) >= (S * 2 == 8 ? 7 : 2)) S *= 2;
  }
  S = std::max(1, std::min(S, std::min(max_s, total_kb)));
  while (S > 1 && (S - 1) * ((total_kb + S - 1) / S) >= total_kb) --S;
  a.S = S;
  a.kb_per_cta = (total_kb + S - 1) / S;
  a.ctas_per_sm = a.n_tiles * S > gs.num_sms ? 2 : 1;
  const Tmap& tw = get_tmap(gs, w, 128, 1);
  const Tmap& tx = get_tmap(gs, xq, a.bn, 1);
  check(b200_gemm_decode_launch(&a, tw.b, tx.b, stream()), "gemm_decode_fp8 launch");
  gs.launches++;
}

int64_t gemm_status() {
  GemmState& gs = gemm_state();
  if (!gs.status.defined()) return 0;
  return gs.status.item<int>();
}
// The GEMM status word itself (one int32 on the device), for callers that copy it to the host with other results.
c10::optional<at::Tensor> gemm_status_tensor() {
  GemmState& gs = gemm_state();
  if (!gs.status.defined()) return c10::nullopt;
  return gs.status;
}
void gemm_clear_tmap_cache() { gemm_state().cache.clear(); }

// out[M, N] = x[M, K] @ w[e(row)]^T for rows sorted by expert (lod), or one group when lod is absent.
// fp8: x / w are uint8 views of e4m3 data, a_scale_t [K/128, stride], w_scale [E, N/128, K/128].
void grouped_gemm(at::Tensor out, const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& lod,
                  const c10::optional<at::Tensor>& bias, const c10::optional<at::Tensor>& a_scale_t,
                  const c10::optional<at::Tensor>& w_scale, int64_t bn) {
  TORCH_CHECK(x.is_cuda() && w.is_cuda() && x.dim() == 2 && (w.dim() == 3 || w.dim() == 2));
  TORCH_CHECK(x.stride(1) == 1 && w.is_contiguous() && out.stride(1) == 1);
  const bool fp8 = x.element_size() == 1;
  TORCH_CHECK(w.element_size() == x.element_size());
  const int E = w.dim() == 3 ? w.size(0) : 1;
  const int N = w.size(-2), K = w.size(-1), M = x.size(0);
  TORCH_CHECK(x.size(1) == K && out.size(0) == M && out.size(1) == N);
  TORCH_CHECK((K * x.element_size()) % 16 == 0 && (x.stride(0) * x.element_size()) % 16 == 0);
  if (M == 0) return;
  if (fp8) TORCH_CHECK(a_scale_t.has_value() && w_scale.has_value() && a_scale_t->stride(1) == 1 && w_scale->is_contiguous());
  c10::cuda::CUDAGuard guard(x.device());
  GemmState& gs = gemm_state();
  std::lock_guard<std::mutex> lk(gs.mu);
  if (gs.num_sms == 0) {
    gs.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    gs.ws = at::empty({16 << 20}, x.options().dtype(at::kFloat));
    gs.counters = at::zeros({1 << 16}, x.options().dtype(at::kInt));
    gs.status = at::zeros({1}, x.options().dtype(at::kInt));
  }
  GroupedGemmArgs a;
  a.out = out.data_ptr(); a.bias = opt_ptr(bias);
  a.lod = lod.has_value() ? lod->data_ptr<int>() : nullptr;
  a.a_scale = fp8 ? a_scale_t->data_ptr<float>() : nullptr;
  a.w_scale = fp8 ? w_scale->data_ptr<float>() : nullptr;
  a.status = gs.status.data_ptr<int>();
  a.M = M; a.N = N; a.K = K; a.E = E; a.ldo = out.stride(0);
  a.a_stride = fp8 ? a_scale_t->stride(0) : 0;
  a.fp8 = fp8; a.fmt = x.scalar_type() == at::kBFloat16 ? 1 : 0; a.out_fmt = out.scalar_type() == at::kBFloat16 ? 1 : 0;
  int b = (int)bn;
  if (b <= 0) {
    // rows per group decide the token tile: decode batches spread thin over many experts
    int per_group = lod.has_value() ? std::max(1, M / std::max(1, E / 4)) : M;
    b = per_group <= 16 ? 16 : per_group <= 32 ? 32 : per_group <= 64 ? 64 : 128;
  }
  a.bn = b;
  int64_t n_tiles = (N + 127) / 128;
  int64_t max_tiles = n_tiles * ((M + b - 1) / b + (lod.has_value() ? E : 0));
  a.grid = (int)std::min<int64_t>(max_tiles, (int64_t)gs.num_sms * (b <= 64 ? 2 : 1));
  at::Tensor w2 = w.dim() == 3 ? w.view({(int64_t)E * N, K}) : w;
  const int eb = x.element_size();
  const Tmap& tw = get_tmap(gs, w2, 128, eb);
  const Tmap& tx = get_tmap(gs, x, b, eb);
  check(b200_grouped_gemm_launch(&a, tw.b, tx.b, stream()), "grouped gemm launch");
}

std::vector<at::Tensor> moe_route(const at::Tensor& logits, const c10::optional<at::Tensor>& bias, int64_t k,
                                  int64_t mode, bool renorm, int64_t n_group, int64_t topk_group, double scale) {
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1);
  auto w = at::empty({logits.size(0), k}, logits.options().dtype(at::kFloat));
  auto ids = at::empty({logits.size(0), k}, logits.options().dtype(at::kInt));
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == at::kFloat && bias->is_contiguous());
  check(b200_moe_route(w.data_ptr<float>(), ids.data_ptr<int>(), logits.data_ptr(),
                       bias.has_value() ? bias->data_ptr<float>() : nullptr, logits.size(0), logits.size(1), k, mode,
                       renorm, n_group, topk_group, (float)scale, logits.stride(0), dtype_code(logits), stream()),
        "moe_route");
  return {w, ids};
}

// Returns x_sorted [T*k, H], pos_of_pair [T*k], lod [E_local + 1].  `state` = int32 [2 * E_local] zero-initialised
// scratch (counts | cursor) owned by the caller.
std::vector<at::Tensor> moe_permute(const at::Tensor& x, const at::Tensor& ids, const c10::optional<at::Tensor>& emap,
                                    int64_t E_local, int64_t E_global, at::Tensor state, int64_t max_rows) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && ids.is_contiguous() && ids.scalar_type() == at::kInt);
  TORCH_CHECK(state.scalar_type() == at::kInt && state.numel() >= 2 * E_local);
  const int64_t T = x.size(0), k = ids.size(1), H = x.size(1);
  if (max_rows <= 0 || max_rows > T * k) max_rows = T * k;  // rows beyond the bound are dropped (pos = -1)
  auto xs = at::empty({max_rows, H}, x.options());
  auto pos = at::empty({T * k}, ids.options());
  auto lod = at::empty({E_local + 1}, ids.options());
  check(b200_moe_permute(xs.data_ptr(), pos.data_ptr<int>(), lod.data_ptr<int>(), state.data_ptr<int>(),
                         state.data_ptr<int>() + E_local, x.data_ptr(), ids.data_ptr<int>(),
                         emap.has_value() ? emap->data_ptr<int>() : nullptr, T, k, H, E_local, E_global, x.stride(0),
                         max_rows, dtype_code(x), stream()),
        "moe_permute", 3);
  return {xs, pos, lod};
}

// (weights [T, k] fp32, ids [T, k] int32) straight from the hidden states: router GEMM + routing in one launch
std::vector<at::Tensor> router_route_small(const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& wbias,
                                           const c10::optional<at::Tensor>& bias, int64_t k, int64_t mode, bool renorm,
                                           int64_t n_group, int64_t topk_group, double scale) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && w.dim() == 2 && w.is_contiguous() && w.scalar_type() == x.scalar_type());
  TORCH_CHECK(w.size(1) == x.size(1));
  if (bias.has_value()) TORCH_CHECK(bias->scalar_type() == at::kFloat && bias->is_contiguous());
  auto ow = at::empty({x.size(0), k}, x.options().dtype(at::kFloat));
  auto oi = at::empty({x.size(0), k}, x.options().dtype(at::kInt));
  check(b200_router_route_small(ow.data_ptr<float>(), oi.data_ptr<int>(), x.data_ptr(), x.stride(0), w.data_ptr(),
                                opt_ptr(wbias), bias.has_value() ? bias->data_ptr<float>() : nullptr, x.size(0),
                                (int)w.size(0), (int)w.size(1), (int)k, (int)mode, renorm, (int)n_group, (int)topk_group,
                                (float)scale, dtype_code(x), stream()), "router_route_small");
  return {ow, oi};
}

at::Tensor router_gemm_small(const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& bias) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && w.dim() == 2 && w.is_contiguous() && w.scalar_type() == x.scalar_type());
  TORCH_CHECK(w.size(1) == x.size(1));
  auto out = at::empty({x.size(0), w.size(0)}, x.options().dtype(at::kFloat));
  check(b200_router_gemm_small(out.data_ptr<float>(), x.data_ptr(), x.stride(0), w.data_ptr(), opt_ptr(bias), x.size(0),
                               (int)w.size(0), (int)w.size(1), dtype_code(x), stream()), "router_gemm_small");
  return out;
}

// Small-batch permute in one launch; with `quant` the rows are written as fp8 with transposed 1x128 scales.
// Returns (x_sorted | q_sorted, pos_of_pair, lod, scale_t or empty).
std::vector<at::Tensor> moe_prepare_small(const at::Tensor& x, const at::Tensor& ids, const c10::optional<at::Tensor>& emap,
                                          int64_t E_local, int64_t E_global, bool quant) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && ids.is_contiguous() && ids.scalar_type() == at::kInt);
  const int64_t T = x.size(0), k = ids.size(1), H = x.size(1), M = T * k;
  TORCH_CHECK(M <= b200_moe_small_pairs() && M >= 1);
  auto xs = at::empty({M, H}, quant ? x.options().dtype(at::kByte) : x.options());
  auto pos = at::empty({M}, ids.options());
  auto lod = at::empty({E_local + 1}, ids.options());
  int64_t stride = std::max<int64_t>(4, (M + 3) / 4 * 4);
  auto st = quant ? at::empty({H / 128, stride}, x.options().dtype(at::kFloat)) : at::empty({0}, x.options().dtype(at::kFloat));
  check(b200_moe_prepare_small(xs.data_ptr(), quant ? st.data_ptr<float>() : nullptr, stride, pos.data_ptr<int>(),
                               lod.data_ptr<int>(), x.data_ptr(), ids.data_ptr<int>(),
                               emap.has_value() ? emap->data_ptr<int>() : nullptr, T, k, H, E_local, E_global, x.stride(0),
                               quant, dtype_code(x), stream()), "moe_prepare_small");
  return {xs, pos, lod, st};
}

// (q uint8 [rows, I], scale_t [I/128, stride]) = fp8(act(h[:, :I]) * h[:, I:])
std::vector<at::Tensor> act_mul_quant_fp8(const at::Tensor& h, int64_t act, const c10::optional<at::Tensor>& rows_valid) {
  TORCH_CHECK(h.dim() == 2 && h.is_contiguous() && h.size(1) % 256 == 0);
  const int64_t rows = h.size(0), I = h.size(1) / 2;
  int64_t stride = std::max<int64_t>(4, (rows + 3) / 4 * 4);
  auto q = at::empty({rows, I}, h.options().dtype(at::kByte));
  auto s = at::empty({I / 128, stride}, h.options().dtype(at::kFloat));
  check(b200_act_mul_quant_fp8(q.data_ptr(), s.data_ptr<float>(), h.data_ptr(), rows, I, stride, act,
                               rows_valid.has_value() ? rows_valid->data_ptr<int>() : nullptr, dtype_code(h), stream()),
        "act_mul_quant_fp8");
  return {q, s};
}

void moe_unpermute(at::Tensor out, const at::Tensor& y_sorted, const at::Tensor& pos, const at::Tensor& w) {
  TORCH_CHECK(out.is_contiguous() && y_sorted.is_contiguous() && w.is_contiguous() && w.scalar_type() == at::kFloat);
  check(b200_moe_unpermute(out.data_ptr(), y_sorted.data_ptr(), pos.data_ptr<int>(), w.data_ptr<float>(), out.size(0),
                           w.size(1), out.size(1), dtype_code(out), stream()),
        "moe_unpermute");
}

// (q uint8 [rows, K], scale_t float [K/128, stride]); rows beyond *rows_valid (device int) are skipped.
std::vector<at::Tensor> quant_fp8_group(const at::Tensor& x, bool ue8m0, const c10::optional<at::Tensor>& rows_valid,
                                        int64_t pad_rows_to) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1);
  const int64_t rows = x.size(0), K = x.size(1);
  int64_t stride = ((rows + pad_rows_to - 1) / pad_rows_to) * pad_rows_to;
  stride = std::max<int64_t>(stride, 4);
  auto q = at::empty({rows, K}, x.options().dtype(at::kByte));
  auto s = at::empty({K / 128, stride}, x.options().dtype(at::kFloat));
  check(b200_quant_fp8_group(q.data_ptr(), s.data_ptr<float>(), x.data_ptr(), rows, K, x.stride(0), stride, ue8m0,
                             rows_valid.has_value() ? rows_valid->data_ptr<int>() : nullptr, dtype_code(x), stream()),
        "quant_fp8_group");
  return {q, s};
}

// ---------------------------------------------------------------------------------------- elementwise
void rmsnorm(at::Tensor out, const at::Tensor& x, const at::Tensor& w, double eps, bool gemma) {
  int H = x.size(-1);
  int64_t rows = x.numel() / H;
  TORCH_CHECK(x.stride(-1) == 1 && out.is_contiguous());
  int64_t xs = x.dim() >= 2 ? x.stride(-2) : H;
  if (x.dim() > 2) TORCH_CHECK(x.is_contiguous());
  check(b200_rmsnorm(out.data_ptr(), x.data_ptr(), nullptr, w.data_ptr(), rows, H, (float)eps, gemma, xs, H,
                     dtype_code(x), stream()), "rmsnorm");
}
void add_rmsnorm(at::Tensor x, at::Tensor residual, const at::Tensor& w, double eps, bool gemma) {
  int H = x.size(-1);
  int64_t rows = x.numel() / H;
  TORCH_CHECK(x.is_contiguous() && residual.is_contiguous());
  check(b200_rmsnorm(x.data_ptr(), x.data_ptr(), residual.data_ptr(), w.data_ptr(), rows, H, (float)eps, gemma, H, H,
                     dtype_code(x), stream()), "add_rmsnorm");
}
void rownorm(at::Tensor out, const at::Tensor& x, const c10::optional<at::Tensor>& z,
             const c10::optional<at::Tensor>& w, double eps, int64_t mode) {
  int D = x.size(-1);
  TORCH_CHECK(x.is_contiguous() && out.is_contiguous());
  check(b200_rownorm(out.data_ptr(), x.data_ptr(), opt_ptr(z), opt_ptr(w), x.numel() / D, D, (float)eps, (int)mode,
                     dtype_code(x), stream()), "rownorm");
}
void act_and_mul(at::Tensor out, const at::Tensor& x, int64_t act) {
  int d = x.size(-1) / 2;
  TORCH_CHECK(x.is_contiguous() && out.is_contiguous());
  check(b200_act_and_mul(out.data_ptr(), x.data_ptr(), x.numel() / (2 * d), d, (int)act, dtype_code(x), stream()),
        "act_and_mul");
}
void quick_gelu(at::Tensor out, const at::Tensor& x) {
  TORCH_CHECK(x.is_contiguous());
  check(b200_quick_gelu(out.data_ptr(), x.data_ptr(), x.numel(), dtype_code(x), stream()), "quick_gelu");
}
void embedding(at::Tensor out, const at::Tensor& ids, const at::Tensor& w, int64_t vocab_start) {
  TORCH_CHECK(ids.scalar_type() == at::kLong && ids.is_contiguous() && w.is_contiguous());
  check(b200_embedding(out.data_ptr(), ids.data_ptr<int64_t>(), w.data_ptr(), ids.numel(), w.size(1), w.size(0),
                       vocab_start, dtype_code(w), stream()), "embedding");
}
void argmax(at::Tensor out, const at::Tensor& logits) {
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && out.scalar_type() == at::kLong);
  // persistent scratch for the per-chunk partial maxima (grown on demand, never inside a capture)
  static at::Tensor sval, sidx;
  const int chunks = 32;
  int64_t need = logits.size(0) * chunks;
  if (!sval.defined() || sval.numel() < need || sval.device() != logits.device()) {
    int64_t n = std::max<int64_t>(need, 4096 * chunks);
    sval = at::empty({n}, logits.options().dtype(at::kFloat));
    sidx = at::empty({n}, logits.options().dtype(at::kInt));
  }
  check(b200_argmax(out.data_ptr<int64_t>(), logits.data_ptr(), logits.size(0), logits.size(1), logits.stride(0),
                    dtype_code(logits), sval.data_ptr<float>(), sidx.data_ptr<int>(), chunks, stream()),
        "argmax", 2);
}

// ---------------------------------------------------------------------------------------- rotary / cache
void qkv_split_norm_rope_cache(at::Tensor q_out, const at::Tensor& qkv, const at::Tensor& positions,
                               const at::Tensor& cos_sin, const c10::optional<at::Tensor>& q_w,
                               const c10::optional<at::Tensor>& k_w, double eps, int64_t Hq, int64_t Hkv, int64_t D,
                               bool neox, bool gemma, const c10::optional<at::Tensor>& kv_cache,
                               const at::Tensor& slots) {
  TORCH_CHECK(qkv.stride(1) == 1 && cos_sin.scalar_type() == at::kFloat && cos_sin.is_contiguous());
  TORCH_CHECK(positions.scalar_type() == at::kLong && slots.scalar_type() == at::kLong);
  int block_size = 0;
  int64_t num_blocks = 0;
  if (kv_cache.has_value()) {
    TORCH_CHECK(kv_cache->is_contiguous() && kv_cache->dim() == 5 && kv_cache->size(2) == Hkv && kv_cache->size(4) == D);
    block_size = kv_cache->size(3);
    num_blocks = kv_cache->size(0);
  }
  check(b200_qkv_split_norm_rope_cache(q_out.data_ptr(), qkv.data_ptr(), positions.data_ptr<int64_t>(),
                                       cos_sin.data_ptr<float>(), opt_ptr(q_w), opt_ptr(k_w), (float)eps,
                                       qkv.size(0), Hq, Hkv, D, cos_sin.size(1), neox, gemma,
                                       kv_cache.has_value() ? kv_cache->data_ptr() : nullptr,
                                       slots.data_ptr<int64_t>(), block_size, num_blocks, cos_sin.size(0),
                                       qkv.stride(0), dtype_code(qkv), stream()), "qkv_split_norm_rope_cache");
}
void rope(at::Tensor q, at::Tensor k, const at::Tensor& positions, const at::Tensor& cos_sin, int64_t D, bool neox) {
  TORCH_CHECK(q.stride(-1) == 1 && k.stride(-1) == 1 && q.dim() == 2 && k.dim() == 2);
  check(b200_rope(q.data_ptr(), k.data_ptr(), positions.data_ptr<int64_t>(), cos_sin.data_ptr<float>(), q.size(0),
                  q.size(1) / D, k.size(1) / D, D, cos_sin.size(1), neox, cos_sin.size(0), q.stride(0), k.stride(0),
                  nullptr, 0, 0, 0, dtype_code(q), stream()), "rope");
}
void mrope(at::Tensor q, at::Tensor k, const at::Tensor& positions3, const at::Tensor& cos_sin, int64_t D,
           std::vector<int64_t> sections, bool interleaved) {
  TORCH_CHECK(positions3.is_contiguous() && positions3.size(0) == 3 && sections.size() == 3);
  check(b200_rope(q.data_ptr(), k.data_ptr(), nullptr, cos_sin.data_ptr<float>(), q.size(0), q.size(1) / D,
                  k.size(1) / D, D, cos_sin.size(1), 1, cos_sin.size(0), q.stride(0), k.stride(0),
                  positions3.data_ptr<int64_t>(), sections[0], sections[1], interleaved, dtype_code(q), stream()),
        "mrope");
}
void reshape_and_cache(const at::Tensor& k, const at::Tensor& v, at::Tensor kv_cache, const at::Tensor& slots) {
  TORCH_CHECK(kv_cache.is_contiguous() && kv_cache.dim() == 5);
  int Hkv = kv_cache.size(2), D = kv_cache.size(4);
  auto k2 = k.reshape({k.size(0), -1}), v2 = v.reshape({v.size(0), -1});
  TORCH_CHECK(k2.stride(1) == 1 && v2.stride(1) == 1 && k2.size(1) == Hkv * D);
  check(b200_reshape_and_cache(k2.data_ptr(), v2.data_ptr(), kv_cache.data_ptr(), slots.data_ptr<int64_t>(),
                               k2.size(0), Hkv, D, kv_cache.size(3), kv_cache.size(0), k2.stride(0), v2.stride(0),
                               dtype_code(k), stream()), "reshape_and_cache");
}
void concat_and_cache_mla(const at::Tensor& kv_c, const at::Tensor& k_pe, at::Tensor cache, const at::Tensor& slots) {
  TORCH_CHECK(cache.is_contiguous() && cache.dim() == 3 && kv_c.stride(-1) == 1 && k_pe.stride(-1) == 1);
  bool fp8 = cache.scalar_type() == at::kByte;
  auto pe = k_pe.reshape({k_pe.size(0), -1});
  check(b200_concat_and_cache_mla(kv_c.data_ptr(), pe.data_ptr(), cache.data_ptr(), slots.data_ptr<int64_t>(),
                                  kv_c.size(0), kv_c.size(1), pe.size(1), cache.size(0) * cache.size(1),
                                  kv_c.stride(0), pe.stride(0), fp8, dtype_code(kv_c), stream()),
        "concat_and_cache_mla");
}
void indexer_k_quant_and_cache(const at::Tensor& k, at::Tensor cache, const at::Tensor& slots, bool ue8m0) {
  TORCH_CHECK(cache.is_contiguous() && cache.scalar_type() == at::kByte && cache.size(-1) == 132 && k.size(1) == 128);
  check(b200_indexer_k_quant_and_cache(k.data_ptr(), cache.data_ptr(), slots.data_ptr<int64_t>(), k.size(0),
                                       cache.size(0) * cache.size(1), ue8m0, k.stride(0), (int)cache.size(1), dtype_code(k),
                                       stream()),
        "indexer_k_quant_and_cache");
}
// Fused indexer operand preparation: returns (q_fp8 [T, H, 128] uint8, w [T, H] float) and writes the key rows.
std::vector<at::Tensor> indexer_prep(const at::Tensor& q, const at::Tensor& k, const at::Tensor& ln_w, const at::Tensor& ln_b,
                                     const at::Tensor& positions, const at::Tensor& cos_sin, const at::Tensor& head_w,
                                     double wscale, at::Tensor cache, const at::Tensor& slots, double eps, bool ue8m0,
                                     int64_t q_lo) {
  // q and head_w hold tokens [q_lo, q_lo + q.size(0)) of the k.size(0) tokens in the batch
  TORCH_CHECK(q.dim() == 3 && q.size(2) == 128 && q.stride(2) == 1 && q.stride(1) == 128 && k.dim() == 2 && k.size(1) == 128 &&
              k.stride(1) == 1 && head_w.dim() == 2 && head_w.stride(1) == 1);
  TORCH_CHECK(q.scalar_type() == k.scalar_type() && q.scalar_type() == ln_w.scalar_type() &&
              q.scalar_type() == ln_b.scalar_type() && q.scalar_type() == head_w.scalar_type());
  TORCH_CHECK(cos_sin.scalar_type() == at::kFloat && cos_sin.is_contiguous() && cos_sin.size(-1) == 64,
              "indexer_prep: rotary dim 64");
  TORCH_CHECK(positions.scalar_type() == at::kLong && slots.scalar_type() == at::kLong && positions.is_contiguous() &&
              slots.is_contiguous());
  TORCH_CHECK(cache.is_contiguous() && cache.scalar_type() == at::kByte && cache.size(-1) == 132);
  const int64_t T = k.size(0), Tq = q.size(0), H = q.size(1);
  TORCH_CHECK(q_lo >= 0 && q_lo + Tq <= T && head_w.size(0) == Tq && head_w.size(1) == H && positions.numel() == T &&
              slots.numel() >= T);
  auto q_out = at::empty({Tq, H, 128}, q.options().dtype(at::kByte));
  auto w_out = at::empty({Tq, H}, q.options().dtype(at::kFloat));
  check(b200_indexer_prep(q.data_ptr(), k.data_ptr(), ln_w.data_ptr(), ln_b.data_ptr(), positions.data_ptr<int64_t>(),
                          cos_sin.data_ptr<float>(), head_w.data_ptr(), (float)wscale, q_out.data_ptr(),
                          w_out.data_ptr<float>(), cache.data_ptr(), slots.data_ptr<int64_t>(), T, (int)H, cos_sin.size(0),
                          cache.size(0) * cache.size(1), q.stride(0), k.stride(0), head_w.stride(0), (float)eps, ue8m0,
                          q_lo, q_lo + Tq, (int)cache.size(1), dtype_code(q), stream()),
        "indexer_prep");
  return {q_out, w_out};
}
// out [M, 576] (bf16 / fp16) <- rows `slots` [M] (int32 global slot ids, negative = zero row) of the latent cache
// [blocks, block_size, 576] (same dtype) or [blocks, block_size, 656] uint8 (fp8_ds_mla rows, de-quantised)
void gather_mla_rows(at::Tensor out, const at::Tensor& cache, const at::Tensor& slots) {
  TORCH_CHECK(out.is_contiguous() && out.dim() == 2 && out.size(1) == 576 && cache.is_contiguous() && cache.dim() == 3);
  TORCH_CHECK(slots.scalar_type() == at::kInt && slots.is_contiguous() && slots.numel() == out.size(0));
  const bool fp8 = cache.scalar_type() == at::kByte;
  if (fp8) {
    TORCH_CHECK(cache.size(2) == 656, "fp8_ds_mla rows are 656 bytes");
  } else {
    TORCH_CHECK(cache.size(2) == 576 && cache.scalar_type() == out.scalar_type());
  }
  check(b200_gather_mla_rows(out.data_ptr(), cache.data_ptr(), slots.data_ptr<int32_t>(), out.size(0),
                             cache.size(0) * cache.size(1), fp8 ? 1 : 0, dtype_code(out), stream()),
        "gather_mla_rows");
}
void convert_req_index_to_global_index(at::Tensor out, const at::Tensor& req_id, const at::Tensor& block_table,
                                       const at::Tensor& idx, int64_t block_size) {
  TORCH_CHECK(req_id.scalar_type() == at::kInt && block_table.scalar_type() == at::kInt && idx.scalar_type() == at::kInt);
  TORCH_CHECK(block_table.is_contiguous() && idx.is_contiguous());
  check(b200_convert_req_index(out.data_ptr<int32_t>(), req_id.data_ptr<int32_t>(), block_table.data_ptr<int32_t>(),
                               idx.data_ptr<int32_t>(), idx.size(0), idx.size(1), block_size, block_table.size(1),
                               block_table.size(0), stream()), "convert_req_index");
}
void copy_blocks(at::Tensor cache, const at::Tensor& src, const at::Tensor& dst) {
  TORCH_CHECK(cache.is_contiguous());
  int64_t bytes = cache.numel() / cache.size(0) * cache.element_size();
  check(b200_copy_blocks(cache.data_ptr(), src.data_ptr<int64_t>(), dst.data_ptr<int64_t>(), src.numel(), bytes,
                         cache.size(0), stream()), "copy_blocks");
}
void merge_attn_states(at::Tensor out, c10::optional<at::Tensor> lse_out, const at::Tensor& o1, const at::Tensor& lse1,
                       const at::Tensor& o2, const at::Tensor& lse2) {
  TORCH_CHECK(o1.is_contiguous() && o2.is_contiguous() && lse1.is_contiguous() && lse2.is_contiguous());
  int D = o1.size(-1);
  check(b200_merge_attn_states(out.data_ptr(), lse_out.has_value() ? lse_out->data_ptr<float>() : nullptr,
                               o1.data_ptr(), lse1.data_ptr<float>(), o2.data_ptr(), lse2.data_ptr<float>(),
                               o1.numel() / D, D, dtype_code(o1), stream()), "merge_attn_states");
}

// ---------------------------------------------------------------------------------------- attention
void paged_attention(at::Tensor out, const at::Tensor& q, const at::Tensor& kv_cache, const at::Tensor& block_tables,
                     const at::Tensor& seq_lens, const at::Tensor& qsl, const c10::optional<at::Tensor>& sinks,
                     const c10::optional<at::Tensor>& ws_o, const c10::optional<at::Tensor>& ws_lse,
                     int64_t max_query_len, int64_t num_splits, int64_t window, double scale, bool decode_layout) {
  TORCH_CHECK(q.is_contiguous() && out.is_contiguous() && kv_cache.is_contiguous() && q.dim() == 3);
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && seq_lens.scalar_type() == at::kInt && qsl.scalar_type() == at::kInt);
  TORCH_CHECK(block_tables.stride(1) == 1);
  if (num_splits > 1) TORCH_CHECK(ws_o.has_value() && ws_lse.has_value());
  int B = seq_lens.size(0);
  check(b200_paged_attention(out.data_ptr(), q.data_ptr(), kv_cache.data_ptr(), block_tables.data_ptr<int>(),
                             seq_lens.data_ptr<int>(), qsl.data_ptr<int>(),
                             sinks.has_value() ? sinks->data_ptr<float>() : nullptr,
                             ws_o.has_value() ? ws_o->data_ptr<float>() : nullptr,
                             ws_lse.has_value() ? ws_lse->data_ptr<float>() : nullptr, q.size(0), B, q.size(1),
                             kv_cache.size(2), q.size(2), kv_cache.size(3), block_tables.stride(0), kv_cache.size(0),
                             max_query_len, num_splits, window, (float)scale, decode_layout, dtype_code(q), stream()),
        "paged_attention", num_splits > 1 ? 2 : 1);
}

// Decode attention on tcgen05 (see api.h); shares the GEMM module's tensor-map cache and status word.
void decode_attention_umma(at::Tensor out, const at::Tensor& q, const at::Tensor& kv_cache, const at::Tensor& block_tables,
                           const at::Tensor& seq_lens, const at::Tensor& qsl, const c10::optional<at::Tensor>& sinks,
                           const c10::optional<at::Tensor>& ws_o, const c10::optional<at::Tensor>& ws_lse,
                           int64_t max_query_len, int64_t num_splits, int64_t window, double scale,
                           bool early_meta) {
  TORCH_CHECK(q.is_contiguous() && out.is_contiguous() && kv_cache.is_contiguous() && q.dim() == 3 && kv_cache.dim() == 5);
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && seq_lens.scalar_type() == at::kInt && qsl.scalar_type() == at::kInt);
  TORCH_CHECK(block_tables.stride(1) == 1 && q.scalar_type() == kv_cache.scalar_type());
  if (num_splits > 1) TORCH_CHECK(ws_o.has_value() && ws_lse.has_value());
  c10::cuda::CUDAGuard guard(q.device());
  GemmState& gs = gemm_state();
  std::lock_guard<std::mutex> lk(gs.mu);
  if (gs.num_sms == 0) {
    gs.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    gs.ws = at::empty({16 << 20}, q.options().dtype(at::kFloat));
    gs.counters = at::zeros({1 << 16}, q.options().dtype(at::kInt));
    gs.status = at::zeros({1}, q.options().dtype(at::kInt));
  }
  const int D = q.size(2);
  at::Tensor flat = kv_cache.view({-1, D});
  const Tmap& tm = get_tmap(gs, flat, 64, 2);
  int B = seq_lens.size(0);
  check(b200_decode_attention_umma(out.data_ptr(), q.data_ptr(), tm.b, block_tables.data_ptr<int>(),
                                   seq_lens.data_ptr<int>(), qsl.data_ptr<int>(),
                                   sinks.has_value() ? sinks->data_ptr<float>() : nullptr,
                                   ws_o.has_value() ? ws_o->data_ptr<float>() : nullptr,
                                   ws_lse.has_value() ? ws_lse->data_ptr<float>() : nullptr, gs.status.data_ptr<int>(),
                                   q.size(0), B, q.size(1), kv_cache.size(2), D, kv_cache.size(3), block_tables.stride(0),
                                   kv_cache.size(0), max_query_len, num_splits, window, (float)scale,
                                   early_meta ? 1 : 0, dtype_code(q), stream()), "decode_attention_umma");
}

extern at::Tensor g_kernel_trace;
// Paged GQA prefill attention on tcgen05 (head_dim 128): q [T, Hq, 128], kv_cache [blocks, 2, Hkv, block_size, 128];
// optional lse [T, Hq] (natural log).
void prefill_attention_umma(at::Tensor out, const at::Tensor& q, const at::Tensor& kv_cache, const at::Tensor& block_tables,
                            const at::Tensor& seq_lens, const at::Tensor& qsl, const c10::optional<at::Tensor>& sinks,
                            const c10::optional<at::Tensor>& lse, int64_t max_query_len, int64_t window, double scale) {
  TORCH_CHECK(q.is_contiguous() && out.is_contiguous() && kv_cache.is_contiguous() && q.dim() == 3 && kv_cache.dim() == 5);
  TORCH_CHECK(q.size(2) == 128 && kv_cache.size(4) == 128 && kv_cache.size(1) == 2 && out.sizes() == q.sizes());
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && seq_lens.scalar_type() == at::kInt && qsl.scalar_type() == at::kInt);
  TORCH_CHECK(block_tables.stride(1) == 1 && q.scalar_type() == kv_cache.scalar_type() && q.scalar_type() == out.scalar_type());
  if (lse.has_value()) TORCH_CHECK(lse->scalar_type() == at::kFloat && lse->is_contiguous() && lse->numel() == q.size(0) * q.size(1));
  if (sinks.has_value()) TORCH_CHECK(sinks->scalar_type() == at::kFloat && sinks->numel() == q.size(1));
  if (q.size(0) == 0) return;
  c10::cuda::CUDAGuard guard(q.device());
  GemmState& gs = gemm_state();
  std::lock_guard<std::mutex> lk(gs.mu);
  if (gs.num_sms == 0) {
    gs.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    gs.ws = at::empty({16 << 20}, q.options().dtype(at::kFloat));
    gs.counters = at::zeros({1 << 16}, q.options().dtype(at::kInt));
    gs.status = at::zeros({1}, q.options().dtype(at::kInt));
  }
  at::Tensor q2 = q.view({q.size(0), q.size(1) * 128});
  at::Tensor flat = kv_cache.view({-1, 128});
  const Tmap& tq = get_tmap(gs, q2, 128, 2);
  const Tmap& tk = get_tmap(gs, flat, 64, 2);
  check(b200_prefill_attention_umma(out.data_ptr(), lse.has_value() ? lse->data_ptr<float>() : nullptr, tq.b, tk.b,
                                    block_tables.data_ptr<int>(), seq_lens.data_ptr<int>(), qsl.data_ptr<int>(),
                                    sinks.has_value() ? sinks->data_ptr<float>() : nullptr, gs.status.data_ptr<int>(),
                                    (int)seq_lens.size(0), (int)q.size(1), (int)kv_cache.size(2), 128, (int)kv_cache.size(3),
                                    (int)block_tables.stride(0), kv_cache.size(0), (int)max_query_len, (int)window,
                                    (float)scale, dtype_code(q),
                                    (g_kernel_trace.defined() &&
                                     g_kernel_trace.numel() >= (int64_t)seq_lens.size(0) * q.size(1) * ((max_query_len + 127) / 128) * 24)
                                        ? reinterpret_cast<unsigned long long*>(g_kernel_trace.data_ptr<int64_t>()) : nullptr,
                                    stream()),
        "prefill_attention_umma");
}

// MLA prefill in the compute-friendly form on tcgen05: q [T, N, 192] (q_nope | rotated q_pe), kv [rows, N * 256]
// (k_nope | v per head: the kv_b_proj output), k_pe [rows, 64] (rotated; may be a strided view), kv_starts / kv_lens
// [B] and qsl [B + 1] int32 -> out [T, N, 128], lse [T, N] (natural log).  Rows of requests without keys are left
// untouched: preset out = 0 and lse = -inf when that can happen.
void mla_prefill_umma(at::Tensor out, const at::Tensor& q, const at::Tensor& kv, const at::Tensor& k_pe,
                      const at::Tensor& kv_starts, const at::Tensor& kv_lens, const at::Tensor& qsl,
                      const c10::optional<at::Tensor>& lse, int64_t max_query_len, bool causal, double scale) {
  TORCH_CHECK(q.is_cuda() && q.is_contiguous() && out.is_contiguous() && q.dim() == 3 && q.size(2) == 192);
  TORCH_CHECK(out.dim() == 3 && out.size(0) == q.size(0) && out.size(1) == q.size(1) && out.size(2) == 128);
  TORCH_CHECK(kv.dim() == 2 && kv.stride(1) == 1 && kv.size(1) == q.size(1) * 256 && (kv.stride(0) * 2) % 16 == 0);
  TORCH_CHECK(k_pe.dim() == 2 && k_pe.stride(1) == 1 && k_pe.size(1) == 64 && k_pe.size(0) == kv.size(0) &&
              (k_pe.stride(0) * 2) % 16 == 0);
  TORCH_CHECK(reinterpret_cast<uintptr_t>(kv.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(k_pe.data_ptr()) % 16 == 0);
  TORCH_CHECK(q.scalar_type() == kv.scalar_type() && q.scalar_type() == k_pe.scalar_type() && q.scalar_type() == out.scalar_type());
  TORCH_CHECK(kv_starts.scalar_type() == at::kInt && kv_lens.scalar_type() == at::kInt && qsl.scalar_type() == at::kInt);
  TORCH_CHECK(kv_starts.is_contiguous() && kv_lens.is_contiguous() && qsl.is_contiguous());
  TORCH_CHECK(kv_starts.numel() == kv_lens.numel() && qsl.numel() == kv_lens.numel() + 1);
  if (lse.has_value()) TORCH_CHECK(lse->scalar_type() == at::kFloat && lse->is_contiguous() && lse->numel() == q.size(0) * q.size(1));
  if (q.size(0) == 0 || kv.size(0) == 0) return;
  c10::cuda::CUDAGuard guard(q.device());
  GemmState& gs = gemm_state();
  std::lock_guard<std::mutex> lk(gs.mu);
  if (gs.num_sms == 0) {
    gs.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    gs.ws = at::empty({16 << 20}, q.options().dtype(at::kFloat));
    gs.counters = at::zeros({1 << 16}, q.options().dtype(at::kInt));
    gs.status = at::zeros({1}, q.options().dtype(at::kInt));
  }
  at::Tensor q2 = q.view({q.size(0), q.size(1) * 192});
  const Tmap& tq = get_tmap(gs, q2, 128, 2);
  const Tmap& tk = get_tmap(gs, kv, 64, 2);
  const Tmap& tp = get_tmap(gs, k_pe, 64, 2);
  const int B = (int)kv_lens.numel();
  check(b200_mla_prefill_umma(out.data_ptr(), lse.has_value() ? lse->data_ptr<float>() : nullptr, tq.b, tk.b, tp.b,
                              kv_starts.data_ptr<int>(), kv_lens.data_ptr<int>(), qsl.data_ptr<int>(),
                              gs.status.data_ptr<int>(), B, (int)q.size(1), (int)max_query_len, causal ? 1 : 0,
                              (float)scale, dtype_code(q),
                              (g_kernel_trace.defined() &&
                               g_kernel_trace.numel() >= (int64_t)B * q.size(1) * ((max_query_len + 127) / 128) * 24)
                                  ? reinterpret_cast<unsigned long long*>(g_kernel_trace.data_ptr<int64_t>()) : nullptr,
                              stream()),
        "mla_prefill_umma");
}

// Dense paged MLA decode on tcgen05: q [T, N, 576], kv [blocks, 64, 576] -> out [T, N, 512].
// Optional phase-trace buffer (int64 [>= CTAs * 24]) for the kernels that support it; an undefined tensor switches it off.
at::Tensor g_kernel_trace;
void set_kernel_trace(const c10::optional<at::Tensor>& t) {
  if (t.has_value()) {
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kLong && t->is_contiguous());
    g_kernel_trace = *t;
  } else {
    g_kernel_trace = at::Tensor();
  }
}

void mla_decode_umma(at::Tensor out, const at::Tensor& q, const at::Tensor& kv, const at::Tensor& block_tables,
                     const at::Tensor& seq_lens, const at::Tensor& qsl, const c10::optional<at::Tensor>& ws_o,
                     const c10::optional<at::Tensor>& ws_lse, int64_t max_query_len, int64_t num_splits, double scale,
                     bool early_meta) {
  TORCH_CHECK(q.is_contiguous() && out.is_contiguous() && kv.is_contiguous() && q.dim() == 3 && kv.dim() == 3);
  TORCH_CHECK(q.size(2) == 576 && kv.size(2) == 576 && out.size(2) == 512 && q.scalar_type() == kv.scalar_type());
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && seq_lens.scalar_type() == at::kInt && qsl.scalar_type() == at::kInt);
  TORCH_CHECK(block_tables.stride(1) == 1);
  if (num_splits > 8 || (num_splits & (num_splits - 1)) != 0)  // 2 / 4 / 8 splits merge inside a cluster
    TORCH_CHECK(ws_o.has_value() && ws_lse.has_value());
  c10::cuda::CUDAGuard guard(q.device());
  GemmState& gs = gemm_state();
  std::lock_guard<std::mutex> lk(gs.mu);
  if (gs.num_sms == 0) {
    gs.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    gs.ws = at::empty({16 << 20}, q.options().dtype(at::kFloat));
    gs.counters = at::zeros({1 << 16}, q.options().dtype(at::kInt));
    gs.status = at::zeros({1}, q.options().dtype(at::kInt));
  }
  at::Tensor flat = kv.view({-1, 576});
  const Tmap& tm = get_tmap(gs, flat, 64, 2);
  int B = seq_lens.size(0);
  check(b200_mla_decode_umma(out.data_ptr(), q.data_ptr(), tm.b, block_tables.data_ptr<int>(), seq_lens.data_ptr<int>(),
                             qsl.data_ptr<int>(), ws_o.has_value() ? ws_o->data_ptr<float>() : nullptr,
                             ws_lse.has_value() ? ws_lse->data_ptr<float>() : nullptr, gs.status.data_ptr<int>(),
                             q.size(0), B, q.size(1), kv.size(1), block_tables.stride(0), kv.size(0), max_query_len,
                             num_splits, (float)scale, early_meta ? 1 : 0, dtype_code(q),
                             (g_kernel_trace.defined() && g_kernel_trace.numel() >= (int64_t)B * num_splits * 64 * 24)
                                 ? reinterpret_cast<unsigned long long*>(g_kernel_trace.data_ptr<int64_t>()) : nullptr,
                             stream()),
        "mla_decode_umma");
}

// q [T, N, 576], kv [blocks, bs, 576] -> out [T, N, 512]; dense (block tables) or sparse (indices [T, topk])
void mla_attention(at::Tensor out, const at::Tensor& q, const at::Tensor& kv, const c10::optional<at::Tensor>& block_tables,
                   const c10::optional<at::Tensor>& seq_lens, const c10::optional<at::Tensor>& qsl,
                   const c10::optional<at::Tensor>& req_of_token, const c10::optional<at::Tensor>& indices,
                   const c10::optional<at::Tensor>& ws_o, const c10::optional<at::Tensor>& ws_lse, int64_t num_splits,
                   double scale) {
  TORCH_CHECK(q.is_contiguous() && out.is_contiguous() && kv.is_contiguous() && q.dim() == 3 && q.size(2) == 576);
  TORCH_CHECK(kv.size(-1) == 576 && out.size(2) == 512);
  const bool sparse = indices.has_value();
  if (sparse) {
    TORCH_CHECK(indices->is_contiguous() && indices->scalar_type() == at::kInt);
  } else {
    TORCH_CHECK(block_tables.has_value() && seq_lens.has_value() && qsl.has_value() && req_of_token.has_value());
  }
  if (num_splits > 1) TORCH_CHECK(ws_o.has_value() && ws_lse.has_value());
  int64_t total_slots = kv.numel() / 576;
  check(b200_mla_attention(out.data_ptr(), q.data_ptr(), kv.data_ptr(),
                           sparse ? nullptr : block_tables->data_ptr<int>(), sparse ? nullptr : seq_lens->data_ptr<int>(),
                           sparse ? nullptr : qsl->data_ptr<int>(), sparse ? nullptr : req_of_token->data_ptr<int>(),
                           sparse ? indices->data_ptr<int>() : nullptr,
                           ws_o.has_value() ? ws_o->data_ptr<float>() : nullptr,
                           ws_lse.has_value() ? ws_lse->data_ptr<float>() : nullptr, q.size(0),
                           sparse ? 0 : seq_lens->size(0), q.size(1), kv.dim() == 3 ? kv.size(1) : 64,
                           sparse ? 0 : block_tables->stride(0), total_slots, sparse ? indices->size(1) : 0, num_splits,
                           (float)scale, dtype_code(q), stream()),
        "mla_attention", num_splits > 1 ? 2 : 1);
}

// logits [T, max_len] fp32 of the lightning indexer; w already carries the per-(token, head) query scale
void indexer_logits(at::Tensor logits, const at::Tensor& q_fp8, const at::Tensor& w, const at::Tensor& k_cache,
                    const at::Tensor& block_tables, const at::Tensor& seq_lens, const at::Tensor& qsl,
                    const at::Tensor& req_of_token, int64_t t0) {
  // req_of_token holds the requests of rows t0 .. t0 + T (a slice of the batch's tokens); t0 = 0 for the whole batch
  TORCH_CHECK(q_fp8.is_contiguous() && q_fp8.element_size() == 1 && q_fp8.size(1) == 64 && q_fp8.size(2) == 128);
  TORCH_CHECK(req_of_token.is_contiguous() && req_of_token.numel() >= q_fp8.size(0) && t0 >= 0);
  TORCH_CHECK(w.is_contiguous() && w.scalar_type() == at::kFloat && k_cache.is_contiguous() && k_cache.size(-1) == 132);
  TORCH_CHECK(logits.is_contiguous() && logits.scalar_type() == at::kFloat && block_tables.stride(1) == 1);
  check(b200_indexer_logits(logits.data_ptr<float>(), q_fp8.data_ptr(), w.data_ptr<float>(), k_cache.data_ptr(),
                            block_tables.data_ptr<int>(), seq_lens.data_ptr<int>(), qsl.data_ptr<int>(),
                            req_of_token.data_ptr<int>(), q_fp8.size(0), seq_lens.size(0), k_cache.size(1),
                            block_tables.stride(0), k_cache.size(0) * k_cache.size(1), logits.size(1), t0, stream()),
        "indexer_logits");
}
// The same logits for prefill-sized batches on tcgen05 (block_size 64): rows are tokens [t0, t0 + q_fp8.size(0)) of the
// batch; only keys [0, n_keys(t)) of a row (rounded up to 128) are written.
void indexer_logits_umma(at::Tensor logits, const at::Tensor& q_fp8, const at::Tensor& w, const at::Tensor& k_cache,
                         const at::Tensor& block_tables, const at::Tensor& seq_lens, const at::Tensor& qsl,
                         int64_t max_query_len, int64_t t0) {
  TORCH_CHECK(q_fp8.is_contiguous() && q_fp8.element_size() == 1 && q_fp8.size(1) == 64 && q_fp8.size(2) == 128);
  TORCH_CHECK(w.is_contiguous() && w.scalar_type() == at::kFloat && w.size(0) == q_fp8.size(0) && w.size(1) == 64);
  TORCH_CHECK(k_cache.is_contiguous() && k_cache.scalar_type() == at::kByte && k_cache.dim() == 3 && k_cache.size(1) == 64 &&
              k_cache.size(2) == 132, "indexer_logits_umma: 64-token pages");
  TORCH_CHECK(logits.is_contiguous() && logits.scalar_type() == at::kFloat && logits.size(0) == q_fp8.size(0));
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && block_tables.stride(1) == 1 && seq_lens.scalar_type() == at::kInt &&
              qsl.scalar_type() == at::kInt && t0 >= 0);
  if (q_fp8.size(0) == 0) return;
  c10::cuda::CUDAGuard guard(q_fp8.device());
  GemmState& gs = gemm_state();
  std::lock_guard<std::mutex> lk(gs.mu);
  if (gs.num_sms == 0) {
    gs.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    gs.ws = at::empty({16 << 20}, w.options().dtype(at::kFloat));
    gs.counters = at::zeros({1 << 16}, w.options().dtype(at::kInt));
    gs.status = at::zeros({1}, w.options().dtype(at::kInt));
  }
  at::Tensor q2 = q_fp8.view({-1, 128});
  if (q2.scalar_type() != at::kByte) q2 = q2.view(at::kByte);
  at::Tensor k2 = k_cache.view({-1, 128});   // a block = 66 rows: 64 key rows, then 2 rows of scales
  const Tmap& tq = get_tmap(gs, q2, 256, 1);
  const Tmap& tk = get_tmap(gs, k2, 64, 1);
  check(b200_indexer_logits_umma(logits.data_ptr<float>(), tq.b, w.data_ptr<float>(), k_cache.data_ptr(), tk.b,
                                 block_tables.data_ptr<int>(), seq_lens.data_ptr<int>(), qsl.data_ptr<int>(),
                                 gs.status.data_ptr<int>(), (int)seq_lens.size(0), (int)max_query_len,
                                 (int)block_tables.stride(0), k_cache.size(0), logits.size(1), t0, t0 + q_fp8.size(0),
                                 stream()),
        "indexer_logits_umma");
}
void topk_rows(at::Tensor out, const at::Tensor& logits, const c10::optional<at::Tensor>& row_len) {
  TORCH_CHECK(out.is_contiguous() && out.scalar_type() == at::kInt && logits.scalar_type() == at::kFloat && logits.stride(1) == 1);
  check(b200_topk_rows(out.data_ptr<int>(), logits.data_ptr<float>(),
                       row_len.has_value() ? row_len->data_ptr<int>() : nullptr, logits.size(0), logits.stride(0),
                       out.size(1), logits.size(1), stream()),
        "topk_rows");
}

// ---------------------------------------------------------------------------------------- peer memory
// Symmetric buffers are plain cudaMalloc allocations shared between the ranks of one node with CUDA
// IPC handles (exchanged by the Python side over the process group).
int64_t peer_alloc(int64_t bytes) {
  void* p = nullptr;
  TORCH_CHECK(cudaMalloc(&p, bytes) == cudaSuccess, "cudaMalloc of the symmetric buffer failed");
  TORCH_CHECK(cudaMemset(p, 0, bytes) == cudaSuccess);
  TORCH_CHECK(cudaDeviceSynchronize() == cudaSuccess);
  return reinterpret_cast<int64_t>(p);
}
void peer_free(int64_t ptr) { cudaFree(reinterpret_cast<void*>(ptr)); }
py::bytes peer_export(int64_t ptr) {
  cudaIpcMemHandle_t h;
  TORCH_CHECK(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(ptr)) == cudaSuccess, "cudaIpcGetMemHandle failed");
  return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
}
int64_t peer_open(const std::string& handle) {
  TORCH_CHECK(handle.size() == sizeof(cudaIpcMemHandle_t));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle.data(), sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  TORCH_CHECK(e == cudaSuccess, "cudaIpcOpenMemHandle failed: ", cudaGetErrorString(e));
  return reinterpret_cast<int64_t>(p);
}
void peer_close(int64_t ptr) { cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr)); }
int64_t allreduce_max_ctas() { return b200_allreduce_max_ctas(); }
int64_t allreduce_flag_bytes() { return b200_allreduce_flag_bytes(); }

// out = sum over ranks of `in`; with `residual` + `weight`: residual += sum, out = rmsnorm(residual) * w.
void oneshot_allreduce(std::vector<int64_t> bufs, const at::Tensor& in, at::Tensor out,
                       const c10::optional<at::Tensor>& residual, const c10::optional<at::Tensor>& weight,
                       at::Tensor epochs, at::Tensor status, int64_t parity_bytes, int64_t flags_offset, int64_t rank,
                       double eps, bool gemma, int64_t grid, int64_t spin_limit) {
  TORCH_CHECK(in.is_contiguous() && out.is_contiguous() && in.dim() == 2);
  TORCH_CHECK(in.numel() * in.element_size() <= parity_bytes, "all-reduce payload exceeds the symmetric buffer");
  if (residual.has_value()) TORCH_CHECK(residual->is_contiguous() && weight.has_value());
  void* ptrs[8] = {nullptr};
  TORCH_CHECK(bufs.size() <= 8);
  for (size_t i = 0; i < bufs.size(); ++i) ptrs[i] = reinterpret_cast<void*>(bufs[i]);
  check(b200_oneshot_allreduce(ptrs, in.data_ptr(), out.data_ptr(), residual.has_value() ? residual->data_ptr() : nullptr,
                               opt_ptr(weight), reinterpret_cast<uint32_t*>(epochs.data_ptr<int>()),
                               status.data_ptr<int>(), parity_bytes, flags_offset, rank, bufs.size(), in.size(0),
                               in.size(1), (float)eps, gemma, grid, (uint32_t)spin_limit, dtype_code(in), stream()),
        "oneshot_allreduce");
}

void ll_allreduce(std::vector<int64_t> bufs, const at::Tensor& in, at::Tensor out,
                  const c10::optional<at::Tensor>& residual, const c10::optional<at::Tensor>& weight, at::Tensor epochs,
                  at::Tensor status, int64_t slot_bytes, int64_t rank, double eps, bool gemma, int64_t grid,
                  int64_t spin_limit, bool skip_push) {
  TORCH_CHECK(in.is_contiguous() && out.is_contiguous() && in.dim() == 2 && in.element_size() == 2);
  if (residual.has_value()) TORCH_CHECK(residual->is_contiguous() && weight.has_value());
  void* ptrs[8] = {nullptr};
  TORCH_CHECK(bufs.size() <= 8);
  for (size_t i = 0; i < bufs.size(); ++i) ptrs[i] = reinterpret_cast<void*>(bufs[i]);
  check(b200_ll_allreduce(ptrs, in.data_ptr(), out.data_ptr(), residual.has_value() ? residual->data_ptr() : nullptr,
                          opt_ptr(weight), reinterpret_cast<uint32_t*>(epochs.data_ptr<int>()), status.data_ptr<int>(),
                          slot_bytes, rank, bufs.size(), in.size(0), in.size(1), (float)eps, gemma, grid,
                          (uint32_t)spin_limit, skip_push ? 1 : 0, dtype_code(in), stream()), "ll_allreduce");
}

at::Tensor tensor_from_ptr(int64_t ptr, std::vector<int64_t> shape, at::ScalarType dtype, int64_t device) {
  auto opts = at::TensorOptions().dtype(dtype).device(at::kCUDA, device);
  return at::from_blob(reinterpret_cast<void*>(ptr), shape, opts);
}

void rs_norm_ag(int64_t stage, int64_t rs_flags, std::vector<int64_t> xfull, std::vector<int64_t> ag_flags,
                int64_t reset_a, int64_t reset_a_n, int64_t reset_b, int64_t reset_b_n,
                const c10::optional<at::Tensor>& residual, const at::Tensor& weight, at::Tensor status, int64_t rank,
                int64_t Tloc, int64_t H, int64_t rs_bn, int64_t n_tiles, int64_t ag_bn, int64_t rows_per_cta,
                int64_t max_tt, double eps, bool gemma, int64_t spin_limit) {
  RsNormArgs a;
  memset(&a, 0, sizeof(a));
  a.stage = reinterpret_cast<const void*>(stage); a.rs_flags = reinterpret_cast<const void*>(rs_flags);
  TORCH_CHECK(xfull.size() <= 8 && xfull.size() == ag_flags.size());
  for (size_t i = 0; i < xfull.size(); ++i) {
    a.xfull[i] = reinterpret_cast<void*>(xfull[i]);
    a.ag_flags[i] = reinterpret_cast<void*>(ag_flags[i]);
  }
  a.reset_a = reinterpret_cast<void*>(reset_a); a.reset_a_n = reset_a_n;
  a.reset_b = reinterpret_cast<void*>(reset_b); a.reset_b_n = reset_b_n;
  if (residual.has_value()) { TORCH_CHECK(residual->is_contiguous()); a.residual = residual->data_ptr(); }
  a.weight = weight.data_ptr(); a.status = status.data_ptr<int>();
  a.rank = rank; a.R = xfull.size(); a.Tloc = Tloc; a.H = H; a.rs_bn = rs_bn; a.n_tiles = n_tiles; a.ag_bn = ag_bn;
  a.rows_per_cta = rows_per_cta; a.max_tt = max_tt; a.gemma = gemma; a.dtype = dtype_code(weight); a.eps = (float)eps;
  a.spin_limit = (unsigned)spin_limit;
  check(b200_rs_norm_ag(&a, stream()), "rs_norm_ag");
}

void sp_wait(int64_t flags, int64_t n_tt, int64_t expect, int64_t spin_limit, at::Tensor status) {
  check(b200_sp_wait(reinterpret_cast<const void*>(flags), n_tt, expect, spin_limit, status.data_ptr<int>(), stream()),
        "sp_wait");
}

// ------------------------------------------------------------------- sampling / GDN / LoRA
template <typename T> const T* optp(const c10::optional<at::Tensor>& t) {
  return t.has_value() ? t->data_ptr<T>() : nullptr;
}

void topk_topp_sample(at::Tensor out, const at::Tensor& logits, const c10::optional<at::Tensor>& temperature,
                      const c10::optional<at::Tensor>& top_k, const c10::optional<at::Tensor>& top_p,
                      const c10::optional<at::Tensor>& noise, int64_t seed, int64_t step) {
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && out.scalar_type() == at::kLong);
  check(b200_topk_topp_sample(out.data_ptr<int64_t>(), logits.data_ptr(), logits.size(0), (int)logits.size(1),
                              logits.stride(0), optp<float>(temperature), optp<int>(top_k), optp<float>(top_p),
                              optp<float>(noise), noise.has_value() ? noise->stride(0) : 0, (uint64_t)seed, (uint64_t)step,
                              dtype_code(logits), stream()), "topk_topp_sample");
}

void repetition_penalty(at::Tensor logits, const at::Tensor& tokens, const at::Tensor& n_tokens, const at::Tensor& penalty,
                        at::Tensor seen) {
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && tokens.scalar_type() == at::kLong && tokens.stride(1) == 1);
  int V = (int)logits.size(1);
  TORCH_CHECK(seen.numel() * seen.element_size() >= logits.size(0) * ((V + 31) / 32) * 4, "seen bitmap too small");
  check(b200_repetition_penalty(logits.data_ptr(), logits.size(0), V, logits.stride(0), tokens.data_ptr<int64_t>(),
                                tokens.stride(0), (int)tokens.size(1), n_tokens.data_ptr<int>(), penalty.data_ptr<float>(),
                                (uint32_t*)seen.data_ptr(), dtype_code(logits), stream()), "repetition_penalty");
}

void rejection_sample(at::Tensor out, const at::Tensor& draft_ids, const at::Tensor& cu_draft, const at::Tensor& target_probs,
                      const c10::optional<at::Tensor>& draft_probs, const at::Tensor& bonus, const at::Tensor& is_greedy,
                      const c10::optional<at::Tensor>& uniform, const c10::optional<at::Tensor>& recover_q, int64_t seed,
                      int64_t step) {
  TORCH_CHECK(target_probs.scalar_type() == at::kFloat && target_probs.is_contiguous() && out.is_contiguous());
  TORCH_CHECK(!draft_probs.has_value() || (draft_probs->scalar_type() == at::kFloat && draft_probs->is_contiguous()));
  TORCH_CHECK(!recover_q.has_value() || recover_q->is_contiguous());
  check(b200_rejection_sample(out.data_ptr<int64_t>(), out.size(0), (int)out.size(1) - 1, draft_ids.data_ptr<int64_t>(),
                              cu_draft.data_ptr<int>(), target_probs.data_ptr<float>(), optp<float>(draft_probs),
                              (int)target_probs.size(1), bonus.data_ptr<int64_t>(), (const uint8_t*)is_greedy.data_ptr(),
                              optp<float>(uniform), optp<float>(recover_q), (uint64_t)seed, (uint64_t)step, stream()),
        "rejection_sample");
}

void causal_conv1d_fwd(at::Tensor out, const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& bias,
                       const at::Tensor& cu, at::Tensor states, const at::Tensor& slots, const at::Tensor& has_init,
                       bool act) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && out.stride(1) == 1 && w.is_contiguous() && states.is_contiguous());
  check(b200_causal_conv1d_fwd(out.data_ptr(), out.stride(0), x.data_ptr(), x.stride(0), w.data_ptr(), opt_ptr(bias),
                               cu.data_ptr<int>(), (int)slots.size(0), states.data_ptr(), slots.data_ptr<int>(),
                               (const uint8_t*)has_init.data_ptr(), (int)x.size(1), (int)w.size(1), act, x.size(0),
                               dtype_code(x), stream()), "causal_conv1d_fwd", 2);
}

void causal_conv1d_update(at::Tensor out, const at::Tensor& x, at::Tensor states, const at::Tensor& w,
                          const c10::optional<at::Tensor>& bias, const at::Tensor& slots, bool act) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && out.stride(1) == 1 && w.is_contiguous() && states.is_contiguous());
  check(b200_causal_conv1d_update(out.data_ptr(), out.stride(0), x.data_ptr(), x.stride(0), states.data_ptr(), w.data_ptr(),
                                  opt_ptr(bias), slots.data_ptr<int>(), x.size(0), (int)x.size(1), (int)w.size(1), act,
                                  dtype_code(x), stream()), "causal_conv1d_update");
}

void gdn_gating(at::Tensor g, at::Tensor beta, const at::Tensor& a, const at::Tensor& b, const at::Tensor& A_log,
                const at::Tensor& dt_bias) {
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && g.is_contiguous() && beta.is_contiguous());
  check(b200_gdn_gating(g.data_ptr<float>(), beta.data_ptr<float>(), a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0),
                        A_log.data_ptr<float>(), dt_bias.data_ptr<float>(), (int)a.size(1), a.size(0), dtype_code(a), stream()),
        "gdn_gating");
}

void gdn_recurrent(at::Tensor out, const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& g,
                   const at::Tensor& beta, at::Tensor states, const at::Tensor& cu, const at::Tensor& slots,
                   const at::Tensor& has_init, double scale, bool l2norm) {
  // q, k [T, Hk, Dk] (same row stride), v [T, Hv, Dv], out [T, Hv, Dv], states [slots, Hv, Dv, Dk] fp32
  TORCH_CHECK(q.dim() == 3 && q.stride(2) == 1 && q.stride(1) == q.size(2) && k.stride(0) == q.stride(0) &&
              k.stride(1) == k.size(2) && v.stride(2) == 1 && v.stride(1) == v.size(2) && out.stride(1) == out.size(2));
  TORCH_CHECK(states.scalar_type() == at::kFloat && states.is_contiguous() && g.is_contiguous() && beta.is_contiguous());
  check(b200_gdn_recurrent(out.data_ptr(), out.stride(0), q.data_ptr(), k.data_ptr(), q.stride(0), v.data_ptr(), v.stride(0),
                           g.data_ptr<float>(), beta.data_ptr<float>(), states.data_ptr<float>(), cu.data_ptr<int>(),
                           slots.data_ptr<int>(), (const uint8_t*)has_init.data_ptr(), (int)slots.size(0), (int)q.size(1),
                           (int)v.size(1), (int)q.size(2), (int)v.size(2), (float)scale, l2norm, dtype_code(q), stream()),
        "gdn_recurrent");
}

void mtp_concat_norm(at::Tensor out, const at::Tensor& embed, const at::Tensor& hidden, const at::Tensor& we,
                     const at::Tensor& wh, const c10::optional<at::Tensor>& pos, double eps) {
  TORCH_CHECK(embed.is_contiguous() && hidden.is_contiguous() && out.is_contiguous());
  check(b200_mtp_concat_norm(out.data_ptr(), embed.data_ptr(), hidden.data_ptr(), we.data_ptr(), wh.data_ptr(),
                             optp<int64_t>(pos), embed.size(0), (int)embed.size(1), (float)eps, dtype_code(embed), stream()),
        "mtp_concat_norm");
}

void sigmoid_gate_mul(at::Tensor out, const at::Tensor& o, const at::Tensor& gate) {
  TORCH_CHECK(o.is_contiguous() && out.is_contiguous() && gate.stride(1) == 1 && o.dim() == 2);
  check(b200_sigmoid_gate_mul(out.data_ptr(), o.data_ptr(), gate.data_ptr(), gate.stride(0), (int)o.size(1), o.size(0),
                              dtype_code(o), stream()), "sigmoid_gate_mul");
}

// ------------------------------------------------------------------- expert-parallel dispatch / combine
struct EpHandle {
  EpArgs a;
  at::Tensor state;  // int32: send_count[R] | recv_count[R] | prev_count[R] | ticket[3] | epoch[1] | status[1]
  at::Tensor sent_slot;
  EpHandle(std::vector<int64_t> peers, std::vector<int64_t> offs, int64_t rank, int64_t cap, int64_t H, int64_t k, int64_t E,
           int64_t row_bytes, int64_t max_tokens, int64_t spin_limit, int64_t device) {
    memset(&a, 0, sizeof(a));
    const int R = (int)peers.size();
    TORCH_CHECK(R <= 8 && offs.size() == 7);
    for (int i = 0; i < R; ++i) a.peer[i] = reinterpret_cast<void*>(peers[i]);
    a.off_x = offs[0]; a.off_scale = offs[1]; a.off_ids = offs[2]; a.off_w = offs[3]; a.off_recv_flag = offs[4];
    a.off_comb = offs[5]; a.off_comb_flag = offs[6];
    auto opts = at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device);
    state = at::zeros({3 * R + 8}, opts);
    sent_slot = at::full({std::max<int64_t>(max_tokens, 1), R}, -1, opts);
    int* sp = state.data_ptr<int>();
    a.send_count = sp; a.recv_count = sp + R; a.prev_count = sp + 2 * R; a.ticket = sp + 3 * R;
    a.epoch = reinterpret_cast<uint32_t*>(sp + 3 * R + 3); a.status = sp + 3 * R + 4;
    a.sent_slot = sent_slot.data_ptr<int>();
    a.rank = rank; a.R = R; a.cap = cap; a.H = H; a.k = k; a.E = E; a.row_bytes = row_bytes; a.spin_limit = (unsigned)spin_limit;
  }
  // `cap` = per-call capacity of one source region (identical on all ranks, >= every rank's token count, <= allocated)
  void dispatch(const at::Tensor& x, const c10::optional<at::Tensor>& scale_t, const at::Tensor& ids, const at::Tensor& w,
                int64_t cap) {
    TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && ids.is_contiguous() && ids.scalar_type() == at::kInt &&
                w.is_contiguous() && w.scalar_type() == at::kFloat && ids.size(1) == a.k);
    TORCH_CHECK(x.size(0) <= cap && cap <= a.cap && x.size(1) * (int64_t)x.element_size() == a.row_bytes);
    TORCH_CHECK((x.stride(0) * x.element_size()) % 16 == 0);
    EpArgs b = a;
    b.x = x.data_ptr(); b.x_row_bytes = x.stride(0) * x.element_size();
    b.x_scale_t = scale_t.has_value() ? scale_t->data_ptr<float>() : nullptr;
    b.scale_stride = scale_t.has_value() ? scale_t->stride(0) : 0;
    b.topk_ids = ids.data_ptr<int>(); b.topk_w = w.data_ptr<float>(); b.T = x.size(0); b.cap = (int)cap;
    check(b200_ep_dispatch(&b, stream()), "ep_dispatch", 2);
  }
  void permute_scales(at::Tensor scale_t, const at::Tensor& recv_scale, const at::Tensor& pos) {
    check(b200_ep_permute_scales(scale_t.data_ptr<float>(), scale_t.stride(0), recv_scale.data_ptr<float>(), pos.data_ptr<int>(),
                                 pos.numel(), a.k, a.H / 128, stream()), "ep_permute_scales");
  }
  void combine(const at::Tensor& y_sorted, const at::Tensor& pos, at::Tensor out, const c10::optional<at::Tensor>& addend,
               int64_t cap) {
    TORCH_CHECK(y_sorted.is_contiguous() && pos.is_contiguous() && out.is_contiguous() && out.size(1) == a.H);
    TORCH_CHECK(pos.numel() == (int64_t)a.R * cap * a.k && cap <= a.cap);
    TORCH_CHECK(!addend.has_value() || (addend->is_contiguous() && addend->scalar_type() == out.scalar_type()));
    EpArgs b = a;
    b.T = out.size(0); b.cap = (int)cap;
    check(b200_ep_combine(&b, y_sorted.data_ptr(), pos.data_ptr<int>(), out.data_ptr(), opt_ptr(addend), dtype_code(out),
                          stream()), "ep_combine", 2);
  }
  int64_t status() { return state[3 * a.R + 4].item<int>(); }
  at::Tensor status_tensor() { return state.slice(0, 3 * a.R + 4, 3 * a.R + 5); }
  at::Tensor recv_count() { return state.slice(0, a.R, 2 * a.R); }
};

void lora_shrink(at::Tensor out, const at::Tensor& x, const at::Tensor& A, const at::Tensor& ids, double scale) {
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && A.dim() == 3 && A.is_contiguous() && out.scalar_type() == at::kFloat &&
              out.is_contiguous() && A.scalar_type() == x.scalar_type());
  check(b200_lora_shrink(out.data_ptr<float>(), x.data_ptr(), x.stride(0), A.data_ptr(), ids.data_ptr<int>(), x.size(0),
                         (int)A.size(1), (int)A.size(2), (float)scale, dtype_code(x), stream()), "lora_shrink");
}

void lora_expand(at::Tensor out, const at::Tensor& h, const at::Tensor& B, const at::Tensor& ids, int64_t offset, bool add) {
  TORCH_CHECK(out.dim() == 2 && out.stride(1) == 1 && B.dim() == 3 && B.is_contiguous() && h.scalar_type() == at::kFloat &&
              h.is_contiguous() && B.scalar_type() == out.scalar_type());
  TORCH_CHECK(offset + B.size(1) <= out.size(1));
  check(b200_lora_expand(out.data_ptr(), out.stride(0), (int)offset, h.data_ptr<float>(), B.data_ptr(), ids.data_ptr<int>(),
                         out.size(0), (int)B.size(1), (int)B.size(2), add, dtype_code(out), stream()), "lora_expand");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("weak_ref_tensor", &weak_ref_tensor);
  m.def("launch_count", &launch_count);
  m.def("gemm", &gemm);
  m.def("gemm_status", &gemm_status);
  m.def("gemm_status_tensor", &gemm_status_tensor);
  m.def("gemm_decode", &gemm_decode);
  m.def("gemm_decode_fp8", &gemm_decode_fp8);
  m.def("gemm_decode_qkv", &gemm_decode_qkv);
  m.def("gemm_decode_w4", &gemm_decode_w4);
  m.def("dequant_w4", &dequant_w4);
  m.def("gemm_int8", &gemm_int8);
  m.def("quant_int8_token", &quant_int8_token);
  m.def("set_gemm_decode_comm", &set_gemm_decode_comm);
  m.def("grouped_gemm", &grouped_gemm);
  m.def("moe_route", &moe_route);
  m.def("moe_permute", &moe_permute, py::arg("x"), py::arg("ids"), py::arg("emap"), py::arg("E_local"),
        py::arg("E_global"), py::arg("state"), py::arg("max_rows") = 0);
  m.def("moe_unpermute", &moe_unpermute);
  m.def("router_gemm_small", &router_gemm_small);
  m.def("router_route_small", &router_route_small);
  m.def("moe_prepare_small", &moe_prepare_small);
  m.def("act_mul_quant_fp8", &act_mul_quant_fp8);
  m.def("moe_small_pairs", []() { return (int64_t)b200_moe_small_pairs(); });
  m.def("quant_fp8_group", &quant_fp8_group);
  m.def("gemm_clear_tmap_cache", &gemm_clear_tmap_cache);
  m.def("rmsnorm", &rmsnorm);
  m.def("add_rmsnorm", &add_rmsnorm);
  m.def("topk_topp_sample", &topk_topp_sample);
  m.def("repetition_penalty", &repetition_penalty);
  m.def("rejection_sample", &rejection_sample);
  m.def("causal_conv1d_fwd", &causal_conv1d_fwd);
  m.def("causal_conv1d_update", &causal_conv1d_update);
  m.def("gdn_gating", &gdn_gating);
  m.def("gdn_recurrent", &gdn_recurrent);
  m.def("mtp_concat_norm", &mtp_concat_norm);
  m.def("sigmoid_gate_mul", &sigmoid_gate_mul);
  m.def("lora_shrink", &lora_shrink);
  m.def("lora_expand", &lora_expand);
  m.def("rownorm", &rownorm);
  m.def("act_and_mul", &act_and_mul);
  m.def("quick_gelu", &quick_gelu);
  m.def("embedding", &embedding);
  m.def("argmax", &argmax);
  m.def("qkv_split_norm_rope_cache", &qkv_split_norm_rope_cache);
  m.def("rope", &rope);
  m.def("mrope", &mrope);
  m.def("reshape_and_cache", &reshape_and_cache);
  m.def("concat_and_cache_mla", &concat_and_cache_mla);
  m.def("indexer_k_quant_and_cache", &indexer_k_quant_and_cache);
  m.def("convert_req_index_to_global_index", &convert_req_index_to_global_index);
  m.def("copy_blocks", &copy_blocks);
  m.def("merge_attn_states", &merge_attn_states);
  m.def("paged_attention", &paged_attention);
  m.def("decode_attention_umma", &decode_attention_umma);
  m.def("mla_decode_umma", &mla_decode_umma);
  m.def("prefill_attention_umma", &prefill_attention_umma);
  m.def("mla_prefill_umma", &mla_prefill_umma);
  m.def("indexer_prep", &indexer_prep);
  m.def("gather_mla_rows", &gather_mla_rows);
  m.def("set_kernel_trace", &set_kernel_trace);
  m.def("mla_decode_max_clusters", [](int64_t R, int64_t S, int64_t dtype) {
    return (int64_t)b200_mla_decode_max_clusters((int)R, (int)S, (int)dtype);
  });
  m.def("mla_attention", &mla_attention);
  m.def("indexer_logits", &indexer_logits);
  m.def("indexer_logits_umma", &indexer_logits_umma);
  m.def("topk_rows", &topk_rows);
  m.def("peer_alloc", &peer_alloc);
  m.def("peer_free", &peer_free);
  m.def("peer_export", &peer_export);
  m.def("peer_open", &peer_open);
  m.def("peer_close", &peer_close);
  m.def("allreduce_max_ctas", &allreduce_max_ctas);
  m.def("allreduce_flag_bytes", &allreduce_flag_bytes);
  m.def("oneshot_allreduce", &oneshot_allreduce);
  m.def("ll_allreduce", &ll_allreduce);
  m.def("set_gemm_comm", &set_gemm_comm);
  m.def("tensor_from_ptr", &tensor_from_ptr);
  m.def("rs_norm_ag", &rs_norm_ag);
  m.def("sp_wait", &sp_wait);
  py::class_<EpHandle>(m, "EpHandle")
      .def(py::init<std::vector<int64_t>, std::vector<int64_t>, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                    int64_t, int64_t>())
      .def("dispatch", &EpHandle::dispatch)
      .def("permute_scales", &EpHandle::permute_scales)
      .def("combine", &EpHandle::combine)
      .def("status", &EpHandle::status)
      .def("status_tensor", &EpHandle::status_tensor)
      .def("recv_count", &EpHandle::recv_count);
}
