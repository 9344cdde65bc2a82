// torch_op.cpp — the drop-in torch-op boundary: `fwd` and `get_scheduler_metadata` with the schemas of
// the reference (kernels/fa4_blackwell.cu:10187-10205; the vLLM `_vllm_fa3_C` surface), registered under
// the namespace given by -DFA3_LIB_NAME (default `_vllm_fa3_C`, as kernels/fa3_hopper.cu:34-36).
// This file only unpacks tensors into the plain-pointer structs of include/fa_b200.h and calls the C ABI.
// PyTorch is used for device memory (outputs, scratch) and the current stream — nothing is computed here.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/all.h>
#include <torch/library.h>

#include <cstdlib>
#include <mutex>
#include <optional>
#include <unordered_map>
#include <vector>

#include "../../include/fa_b200.h"

#ifndef FA3_LIB_NAME
#define FA3_LIB_NAME _vllm_fa3_C
#endif

namespace {

int dtype_code(at::ScalarType t) {
  if (t == at::kBFloat16) return FA_DT_BF16;
  if (t == at::kHalf) return FA_DT_FP16;
  if (t == at::kFloat8_e4m3fn) return FA_DT_FP8_E4M3;
  return -1;
}

const int32_t* i32(const std::optional<at::Tensor>& t, const char* name) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->scalar_type() == at::kInt && t->is_contiguous() && t->is_cuda(), name,
              " must be a contiguous int32 CUDA tensor");
  return t->data_ptr<int32_t>();
}

// Environment switches, read once when the library is loaded:
//   FA_B200_ROUTE=<0..3>        force a kernel family (FA_ROUTE_*), for testing and A/B runs
//   FA_B200_CHECK_STATUS=1      synchronise after every call and read the device status word
struct EnvConfig {
  int route = FA_ROUTE_AUTO;
  bool check_status = false;
  EnvConfig() {
    if (const char* r = std::getenv("FA_B200_ROUTE")) route = std::atoi(r);
    const char* v = std::getenv("FA_B200_CHECK_STATUS");
    check_status = v && v[0] && v[0] != '0';
  }
};
const EnvConfig& env_config() {
  static const EnvConfig cfg;
  return cfg;
}

// Scratch for fa_b200_fwd, kept per (device, stream) and reused: its 256-byte header is zeroed once when the
// buffer is made and every call leaves it zero again (FA_FLAG_WORKSPACE_CLEAN), so a call costs neither an
// allocation nor a memset.  Calls on one stream run one after the other, which is what sharing a buffer needs.
// Requests above kCacheLimit are served by a plain allocation instead.
constexpr int64_t kCacheLimit = 64ll << 20;
struct WsKey {
  int device;
  cudaStream_t stream;
  bool operator==(const WsKey& o) const { return device == o.device && stream == o.stream; }
};
struct WsKeyHash {
  size_t operator()(const WsKey& k) const { return std::hash<const void*>()(k.stream) * 31u + (size_t)k.device; }
};
std::mutex g_ws_mu;
std::unordered_map<WsKey, at::Tensor, WsKeyHash> g_ws_cache;

at::Tensor cached_workspace(const at::Tensor& like, cudaStream_t stream, int64_t bytes, bool* clean) {
  if (bytes > kCacheLimit) {
    *clean = false;
    return at::empty({bytes}, like.options().dtype(at::kByte));
  }
  const WsKey key{(int)like.get_device(), stream};
  std::lock_guard<std::mutex> lk(g_ws_mu);
  auto it = g_ws_cache.find(key);
  if (it == g_ws_cache.end() || it->second.numel() < bytes) {
    const int64_t cap = std::max<int64_t>(bytes, 1 << 20);
    at::Tensor t = at::zeros({cap}, like.options().dtype(at::kByte));   // zero-filled on the current stream
    if (it == g_ws_cache.end()) it = g_ws_cache.emplace(key, t).first;
    else it->second = t;
  }
  *clean = true;
  return it->second;
}
void drop_cached_workspace(const at::Tensor& like, cudaStream_t stream) {
  std::lock_guard<std::mutex> lk(g_ws_mu);
  g_ws_cache.erase(WsKey{(int)like.get_device(), stream});
}

void check_rc(int rc, const char* what) {
  if (rc == FA_OK) return;
  TORCH_CHECK(false, "fa_b200: ", what, ": ", fa_b200_strerror(rc),
              rc == FA_ERR_LAUNCH ? " — " : "", rc == FA_ERR_LAUNCH ? fa_b200_last_cuda_error() : "");
}

// Mirrors mha_fwd (kernels/fa4_blackwell.cu:10081-10173): same arguments, same return
// {out, softmax_lse, empty, empty}; unsupported configurations raise with "unsupported" in the text.
std::vector<at::Tensor> mha_fwd(
    at::Tensor q, at::Tensor k, at::Tensor v,
    std::optional<at::Tensor> k_new, std::optional<at::Tensor> v_new, std::optional<at::Tensor> q_v,
    std::optional<at::Tensor> out_,
    std::optional<at::Tensor> cu_seqlens_q, std::optional<at::Tensor> cu_seqlens_k,
    std::optional<at::Tensor> cu_seqlens_k_new,
    std::optional<at::Tensor> seqused_q, std::optional<at::Tensor> seqused_k,
    std::optional<int64_t> max_seqlen_q, std::optional<int64_t> max_seqlen_k,
    std::optional<at::Tensor> page_table, std::optional<at::Tensor> kv_batch_idx,
    std::optional<at::Tensor> leftpad_k,
    std::optional<at::Tensor> rotary_cos, std::optional<at::Tensor> rotary_sin,
    std::optional<at::Tensor> seqlens_rotary,
    std::optional<at::Tensor> q_descale, std::optional<at::Tensor> k_descale, std::optional<at::Tensor> v_descale,
    double softmax_scale, bool is_causal, int64_t window_size_left, int64_t window_size_right,
    double softcap, bool is_rotary_interleaved,
    std::optional<at::Tensor> scheduler_metadata, int64_t num_splits, std::optional<bool> pack_gqa,
    int64_t sm_margin,
    std::optional<at::Tensor> s_aux, int64_t cp_world_size, int64_t cp_rank,
    std::optional<at::Tensor> cp_tot_seqused_k) {
  TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda(), "fa_b200: q, k, v must be CUDA tensors");
  const at::cuda::OptionalCUDAGuard guard(q.device());
  TORCH_CHECK(q.dim() == 3, "fa_b200: unsupported config (q must be (total_q, hq, hd))");
  TORCH_CHECK(cu_seqlens_q.has_value(), "fa_b200: unsupported config (cu_seqlens_q is required)");
  TORCH_CHECK(!q_v.has_value() && !seqused_q.has_value() && cp_world_size <= 1,
              "fa_b200: unsupported config (q_v / seqused_q / context-parallel)");
  TORCH_CHECK(k_new.has_value() == v_new.has_value(), "fa_b200: unsupported config (k_new and v_new come together)");
  TORCH_CHECK(rotary_cos.has_value() == rotary_sin.has_value() && (!rotary_cos.has_value() || k_new.has_value()),
              "fa_b200: unsupported config (rotary_cos and rotary_sin come together, and only with k_new / v_new)");
  // A cache laid out (batch_cache, seqlen_cache, hkv, d) without a page table is a paged cache with one page per row
  // of the batch: page b (or kv_batch_idx[b]) belongs to sequence b.
  bool paged = page_table.has_value();
  if (!paged && k.dim() == 4) {
    TORCH_CHECK(seqused_k.has_value(), "fa_b200: unsupported config (a (batch, seqlen, heads, dim) cache needs seqused_k)");
    const int64_t nb = cu_seqlens_q->numel() - 1;
    page_table = kv_batch_idx.has_value()
                     ? kv_batch_idx->to(at::kInt).reshape({nb, 1}).contiguous()
                     : at::arange(nb, seqused_k->options().dtype(at::kInt)).reshape({nb, 1});
    paged = true;
  } else {
    TORCH_CHECK(!kv_batch_idx.has_value(), "fa_b200: unsupported config (kv_batch_idx with a paged or packed cache)");
  }
  TORCH_CHECK(k.dim() == (paged ? 4 : 3) && v.dim() == k.dim(),
              "fa_b200: unsupported config (k/v rank does not match paged=", paged, ")");
  TORCH_CHECK(q.stride(2) == 1 && k.stride(-1) == 1 && v.stride(-1) == 1,
              "fa_b200: unsupported config (the last dim of q, k, v must be contiguous)");

  FaFwdParams p{};
  p.total_q = (int)q.size(0); p.hq = (int)q.size(1); p.hd = (int)q.size(2);
  p.hkv = paged ? (int)k.size(2) : (int)k.size(1);
  p.hdv = paged ? (int)v.size(3) : (int)v.size(2);
  p.q_dtype = dtype_code(q.scalar_type());
  p.kv_dtype = dtype_code(k.scalar_type());
  TORCH_CHECK(p.q_dtype >= 0 && p.kv_dtype >= 0 && k.scalar_type() == v.scalar_type(),
              "fa_b200: unsupported config (dtype q=", q.scalar_type(), " k=", k.scalar_type(), ")");
  // `out` is q's type (bf16 for e4m3 q); a caller-supplied float32 `out` asks for the normalised result in fp32,
  // the form a partial result has before a merge
  auto out_type = q.scalar_type() == at::kFloat8_e4m3fn ? at::kBFloat16 : q.scalar_type();
  if (out_.has_value() && out_->scalar_type() == at::kFloat) out_type = at::kFloat;
  p.out_dtype = out_type == at::kFloat ? FA_DT_FP32 : dtype_code(out_type);

  at::Tensor out = out_.has_value() ? *out_ : at::empty({p.total_q, p.hq, p.hdv}, q.options().dtype(out_type));
  TORCH_CHECK(out.scalar_type() == out_type && out.dim() == 3 && out.size(0) == p.total_q && out.size(1) == p.hq &&
                  out.size(2) == p.hdv && out.stride(2) == 1,
              "fa_b200: unsupported config (out has the wrong shape, dtype or layout)");
  at::Tensor lse = at::empty({p.hq, p.total_q}, q.options().dtype(at::kFloat));

  p.q = q.data_ptr(); p.k = k.data_ptr(); p.v = v.data_ptr(); p.out = out.data_ptr();
  p.lse = lse.data_ptr<float>();
  p.q_row_stride = q.stride(0); p.q_head_stride = q.stride(1);
  p.o_row_stride = out.stride(0); p.o_head_stride = out.stride(1);
  if (paged) {
    p.k_page_stride = k.stride(0); p.k_row_stride = k.stride(1); p.k_head_stride = k.stride(2);
    p.v_page_stride = v.stride(0); p.v_row_stride = v.stride(1); p.v_head_stride = v.stride(2);
    p.page_size = (int)k.size(1); p.num_pages = (int)k.size(0);
    p.page_table = i32(page_table, "page_table");
    TORCH_CHECK(page_table->dim() == 2, "fa_b200: page_table must be (batch, max_pages)");
    p.page_table_stride = (int)page_table->stride(0);
    TORCH_CHECK(seqused_k.has_value(), "fa_b200: unsupported config (paged KV needs seqused_k)");
  } else {
    p.k_row_stride = k.stride(0); p.k_head_stride = k.stride(1);
    p.v_row_stride = v.stride(0); p.v_head_stride = v.stride(1);
    p.total_k = (int)k.size(0);
    TORCH_CHECK(cu_seqlens_k.has_value(), "fa_b200: unsupported config (non-paged KV needs cu_seqlens_k)");
  }
  p.cu_seqlens_q = i32(cu_seqlens_q, "cu_seqlens_q");
  p.cu_seqlens_k = i32(cu_seqlens_k, "cu_seqlens_k");
  p.seqused_k = i32(seqused_k, "seqused_k");
  p.leftpad_k = i32(leftpad_k, "leftpad_k");
  p.batch = (int)cu_seqlens_q->numel() - 1;
  // The two maxima are optional in the schema (the reference derives them when absent, through a device-to-host
  // copy of cu_seqlens, kernels/fa4_blackwell.cu:9427-9431).  Any upper bound serves: the kernels read the true lengths on
  // the device, so the bounds come from the tensor shapes, without a device-to-host copy.
  p.max_seqlen_q = max_seqlen_q.has_value() ? (int)*max_seqlen_q : p.total_q;
  p.max_seqlen_k = max_seqlen_k.has_value() ? (int)*max_seqlen_k
                   : paged               ? (int)(page_table->size(1) * k.size(1))
                                         : (int)k.size(0);

  // ---- k_new / v_new: append to the cache in place (and rotate) before the attention call ----
  at::Tensor q_rot, seq_after, cu_new, kn, vn, rcos, rsin;
  if (k_new.has_value()) {
    TORCH_CHECK(paged && seqused_k.has_value(), "fa_b200: unsupported config (k_new / v_new need a paged or (batch, seqlen) cache and seqused_k)");
    TORCH_CHECK(!leftpad_k.has_value(), "fa_b200: unsupported config (k_new / v_new with leftpad_k)");
    kn = *k_new; vn = *v_new;
    TORCH_CHECK(kn.scalar_type() == k.scalar_type() && vn.scalar_type() == v.scalar_type() && kn.is_cuda() && vn.is_cuda(),
                "fa_b200: unsupported config (k_new / v_new must have the cache's dtype)");
    int64_t max_new = 0;
    if (kn.dim() == 4) {   // (batch, seqlen_new, hkv, d): every sequence gets seqlen_new keys
      const int64_t s_new = kn.size(1);
      TORCH_CHECK(kn.size(0) == p.batch && vn.dim() == 4, "fa_b200: unsupported config (k_new batch size)");
      cu_new = at::arange(0, (p.batch + 1) * s_new, s_new, seqused_k->options().dtype(at::kInt));
      kn = kn.reshape({p.batch * s_new, kn.size(2), kn.size(3)});
      vn = vn.reshape({p.batch * s_new, vn.size(2), vn.size(3)});
      max_new = s_new;
    } else {
      TORCH_CHECK(kn.dim() == 3 && vn.dim() == 3 && cu_seqlens_k_new.has_value(),
                  "fa_b200: unsupported config (packed k_new needs cu_seqlens_k_new)");
      cu_new = *cu_seqlens_k_new;
      max_new = kn.size(0);
    }
    TORCH_CHECK(kn.stride(2) == 1 && vn.stride(2) == 1 && kn.size(1) == p.hkv && kn.size(2) == p.hd && vn.size(2) == p.hdv,
                "fa_b200: unsupported config (k_new / v_new shape or layout)");
    std::optional<at::Tensor> cu_new_o(cu_new);
    FaAppendParams ap{};
    ap.k_new = kn.data_ptr(); ap.v_new = vn.data_ptr(); ap.k_cache = k.data_ptr(); ap.v_cache = v.data_ptr();
    ap.kn_row_stride = kn.stride(0); ap.kn_head_stride = kn.stride(1);
    ap.vn_row_stride = vn.stride(0); ap.vn_head_stride = vn.stride(1);
    ap.k_page_stride = p.k_page_stride; ap.k_row_stride = p.k_row_stride; ap.k_head_stride = p.k_head_stride;
    ap.v_page_stride = p.v_page_stride; ap.v_row_stride = p.v_row_stride; ap.v_head_stride = p.v_head_stride;
    ap.cu_seqlens_k_new = i32(cu_new_o, "cu_seqlens_k_new");
    ap.cu_seqlens_q = p.cu_seqlens_q;
    ap.seqused_k = p.seqused_k;
    seq_after = at::empty_like(*seqused_k);
    ap.seqused_k_out = seq_after.data_ptr<int32_t>();
    ap.page_table = p.page_table; ap.page_table_stride = p.page_table_stride; ap.page_size = p.page_size;
    ap.batch = p.batch; ap.total_new = (int)kn.size(0); ap.total_q = p.total_q;
    ap.hq = p.hq; ap.hkv = p.hkv; ap.hd = p.hd; ap.hdv = p.hdv;
    ap.kv_dtype = p.kv_dtype; ap.q_dtype = p.q_dtype == FA_DT_FP16 ? FA_DT_FP16 : FA_DT_BF16;
    if (rotary_cos.has_value()) {
      TORCH_CHECK(p.q_dtype != FA_DT_FP8_E4M3, "fa_b200: unsupported config (rotary with e4m3 queries)");
      rcos = rotary_cos->to(q.scalar_type()).contiguous();
      rsin = rotary_sin->to(q.scalar_type()).contiguous();
      TORCH_CHECK(rcos.dim() == 2 && rsin.sizes() == rcos.sizes(), "fa_b200: unsupported config (rotary tables must be (seqlen_ro, rotary_dim/2))");
      q_rot = at::empty(q.sizes(), q.options());
      ap.q = q.data_ptr(); ap.q_out = q_rot.data_ptr();
      ap.q_row_stride = q.stride(0); ap.q_head_stride = q.stride(1);
      ap.qo_row_stride = q_rot.stride(0); ap.qo_head_stride = q_rot.stride(1);
      ap.rotary_cos = rcos.data_ptr(); ap.rotary_sin = rsin.data_ptr();
      ap.rotary_dim = 2 * (int)rcos.size(1);
      ap.seqlens_rotary = i32(seqlens_rotary, "seqlens_rotary");
      ap.rotary_interleaved = is_rotary_interleaved ? 1 : 0;
      ap.q_positions_advance = (is_causal || window_size_left >= 0 || window_size_right >= 0) ? 1 : 0;
    }
    const int arc = fa_b200_append_kv(&ap, (fa_stream_t)at::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(arc != FA_ERR_UNSUPPORTED, "fa_b200: unsupported config (k_new / v_new / rotary shapes or alignment)");
    check_rc(arc, "append_kv");
    p.seqused_k = seq_after.data_ptr<int32_t>();
    if (q_rot.defined()) { p.q = q_rot.data_ptr(); p.q_row_stride = q_rot.stride(0); p.q_head_stride = q_rot.stride(1); }
    p.max_seqlen_k = (int)std::min<int64_t>((int64_t)p.max_seqlen_k + max_new, page_table->size(1) * (int64_t)p.page_size);
  }

  // fp8 descales: (batch, hkv) float tables or one-element tensors, materialised as (batch, hkv) fp32
  at::Tensor qd, kd, vd;
  auto descale = [&](const std::optional<at::Tensor>& d, at::Tensor& keep, const char* name) -> const float* {
    if (!d.has_value()) return nullptr;
    TORCH_CHECK(d->is_cuda(), name, " must be a CUDA tensor");
    at::Tensor f = d->to(at::kFloat);
    if (f.numel() == 1) f = f.reshape({1, 1});
    TORCH_CHECK(f.dim() == 2 && (f.size(0) == p.batch || f.size(0) == 1) && (f.size(1) == p.hkv || f.size(1) == 1),
                name, " must be (batch, hkv) or a single element");
    keep = f.expand({p.batch, p.hkv}).contiguous();
    return keep.data_ptr<float>();
  };
  p.q_descale = descale(q_descale, qd, "q_descale");
  p.k_descale = descale(k_descale, kd, "k_descale");
  p.v_descale = descale(v_descale, vd, "v_descale");
  p.descale_batch_stride = p.hkv; p.descale_head_stride = 1;

  at::Tensor s_aux_f;
  if (s_aux.has_value()) {
    s_aux_f = s_aux->to(at::kFloat).contiguous();
    TORCH_CHECK(s_aux_f.numel() == p.hq, "fa_b200: s_aux must have one logit per q head");
    p.s_aux = s_aux_f.data_ptr<float>();
  }
  // A tensor shorter than the header is a placeholder (the reference's op returns zeros({1}),
  // kernels/fa4_blackwell.cu:10182) and is ignored; anything longer must be this library's metadata for this very
  // problem: the length is checked on the host, the header on the device.
  p.scheduler_metadata = i32(scheduler_metadata, "scheduler_metadata");
  if (scheduler_metadata.has_value() && scheduler_metadata->numel() < 16) p.scheduler_metadata = nullptr;
  if (p.scheduler_metadata) p.scheduler_metadata_len = (int)scheduler_metadata->numel();

  p.softmax_scale = (float)softmax_scale; p.softcap = (float)softcap;
  p.is_causal = is_causal ? 1 : 0;
  p.window_left = (int)window_size_left; p.window_right = (int)window_size_right;
  p.num_splits = (int)num_splits; p.sm_margin = (int)sm_margin;
  const EnvConfig& env = env_config();
  p.route = env.route;

  const size_t ws_bytes = fa_b200_fwd_workspace_bytes(&p);
  auto stream = at::cuda::getCurrentCUDAStream();
  bool clean = false;
  at::Tensor ws = cached_workspace(q, stream.stream(), (int64_t)ws_bytes, &clean);
  if (clean) p.flags |= FA_FLAG_WORKSPACE_CLEAN;
  const int rc = fa_b200_fwd(&p, ws.data_ptr(), (size_t)ws.numel(), (fa_stream_t)stream.stream());
  if (rc == FA_ERR_UNSUPPORTED) {
    TORCH_CHECK(false, "fa_b200: unsupported config (hd=", p.hd, " hdv=", p.hdv, " paged=", paged,
                " page_size=", p.page_size, " q dtype=", q.scalar_type(), " kv dtype=", k.scalar_type(), ")");
  }
  check_rc(rc, "fwd");
  if (env.check_status) {
    uint32_t detail = 0;
    const int st = fa_b200_check_status(ws.data_ptr(), (fa_stream_t)stream.stream(), &detail);
    if (st != FA_OK) drop_cached_workspace(q, stream.stream());   // its header is no longer clean
    TORCH_CHECK(st == FA_OK, "fa_b200: ", fa_b200_strerror(st), " (detail=", detail, ")");
  }
  at::Tensor empty = at::empty({0}, q.options().dtype(at::kFloat));
  return {out, lse, empty, empty};
}

// Mirrors mha_fwd_get_scheduler_metadata (kernels/fa4_blackwell.cu:10175-10183): same arguments; returns an
// int32 tensor that `fwd` accepts back through `scheduler_metadata`.
at::Tensor mha_fwd_get_scheduler_metadata(
    int64_t batch_size, int64_t max_seqlen_q, int64_t max_seqlen_k, int64_t num_heads, int64_t num_heads_k,
    int64_t headdim, int64_t headdim_v, at::ScalarType qkv_dtype, at::Tensor seqused_k,
    std::optional<at::Tensor> cu_seqlens_q, std::optional<at::Tensor> cu_seqlens_k,
    std::optional<at::Tensor> cu_seqlens_k_new, std::optional<at::Tensor> seqused_q,
    std::optional<at::Tensor> leftpad_k, std::optional<int64_t> page_size, int64_t max_seqlen_k_new,
    bool is_causal, int64_t window_size_left, int64_t window_size_right, bool has_softcap, int64_t num_splits,
    std::optional<bool> pack_gqa, int64_t sm_margin) {
  TORCH_CHECK(seqused_k.is_cuda(), "fa_b200: seqused_k must be a CUDA tensor");
  const at::cuda::OptionalCUDAGuard guard(seqused_k.device());
  FaSchedParams sp{};
  std::optional<at::Tensor> su(seqused_k);
  sp.seqused_k = i32(su, "seqused_k");
  sp.cu_seqlens_q = i32(cu_seqlens_q, "cu_seqlens_q");
  sp.cu_seqlens_k = i32(cu_seqlens_k, "cu_seqlens_k");
  sp.leftpad_k = i32(leftpad_k, "leftpad_k");
  sp.batch = (int)batch_size; sp.max_seqlen_q = (int)max_seqlen_q; sp.max_seqlen_k = (int)max_seqlen_k;
  sp.hq = (int)num_heads; sp.hkv = (int)num_heads_k; sp.hd = (int)headdim; sp.hdv = (int)headdim_v;
  sp.qkv_dtype = dtype_code(qkv_dtype);
  TORCH_CHECK(sp.qkv_dtype >= 0, "fa_b200: unsupported config (qkv_dtype)");
  sp.page_size = page_size.has_value() ? (int)*page_size : 0;
  sp.is_causal = is_causal; sp.window_left = (int)window_size_left; sp.window_right = (int)window_size_right;
  sp.has_softcap = has_softcap; sp.num_splits = (int)num_splits; sp.sm_margin = (int)sm_margin;
  const int len = fa_b200_scheduler_metadata_len(&sp);
  at::Tensor md = at::empty({len}, seqused_k.options().dtype(at::kInt));
  auto stream = at::cuda::getCurrentCUDAStream();
  check_rc(fa_b200_get_scheduler_metadata(&sp, md.data_ptr<int32_t>(), (fa_stream_t)stream.stream()),
           "get_scheduler_metadata");
  return md;
}

}  // namespace

TORCH_LIBRARY(FA3_LIB_NAME, m) {
  m.def("fwd(Tensor! q, Tensor k, Tensor v, Tensor? k_new, Tensor? v_new, Tensor? q_v, "
        "Tensor!? out, Tensor? cu_seqlens_q, Tensor? cu_seqlens_k, Tensor? cu_seqlens_k_new, "
        "Tensor? seqused_q, Tensor? seqused_k, int? max_seqlen_q, int? max_seqlen_k, "
        "Tensor? page_table, Tensor? kv_batch_idx, Tensor? leftpad_k, Tensor? rotary_cos, "
        "Tensor? rotary_sin, Tensor? seqlens_rotary, Tensor? q_descale, Tensor? k_descale, "
        "Tensor? v_descale, float softmax_scale, bool is_causal, int window_size_left, "
        "int window_size_right, float softcap, bool is_rotary_interleaved, "
        "Tensor? scheduler_metadata, int num_splits, bool? pack_gqa, int sm_margin, "
        "Tensor? s_aux, int cp_world_size, int cp_rank, Tensor? cp_tot_seqused_k) -> Tensor[]");
  m.impl("fwd", torch::kCUDA, &mha_fwd);
  m.def("get_scheduler_metadata(int batch_size, int max_seqlen_q, int max_seqlen_k, "
        "int num_heads, int num_heads_k, int headdim, int headdim_v, ScalarType qkv_dtype, "
        "Tensor seqused_k, Tensor? cu_seqlens_q, Tensor? cu_seqlens_k, Tensor? cu_seqlens_k_new, "
        "Tensor? seqused_q, Tensor? leftpad_k, int? page_size, int max_seqlen_k_new, "
        "bool is_causal, int window_size_left, int window_size_right, bool has_softcap, "
        "int num_splits, bool? pack_gqa, int sm_margin) -> Tensor");
  m.impl("get_scheduler_metadata", torch::kCUDA, &mha_fwd_get_scheduler_metadata);
}
