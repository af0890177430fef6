// PyTorch face of libstx.so: registers, under the reference's own names, the custom class
// `torch.classes.sparse_mlp.WeightCache` and the operators `torch.ops.sparse_mlp.forward`
// and `torch.ops.sparse_mlp.approx_topk_threshold` (reference: TORCH_LIBRARY(sparse_mlp, m),
// sparse_transformers/csrc/sparse_mlp_op.cpp:195-209).  Every method forwards to the C ABI
// in include/stx.h on the current CUDA stream; there is no CPU implementation here, and
// CPU tensors are rejected (weights) or moved to the cache's device (masks).
#include <torch/custom_class.h>
#include <torch/script.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <cuda_runtime.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <string>

#include "stx.h"

namespace stxb {

static void check(int rc, const char* where) {
  if (rc == STX_OK) return;
  const char* msg = stx_last_error();
  // Same texts as the reference for the two user-visible failures
  // (weight_cache.h:117-118 "No active weights", :364 "Cache is not valid").
  TORCH_CHECK(false, (msg && *msg) ? msg : stx_status_string(rc), " [", where, "]");
}

static int to_stx_dtype(c10::ScalarType t) {
  switch (t) {
    case c10::kFloat: return STX_F32;
    case c10::kHalf: return STX_F16;
    case c10::kBFloat16: return STX_BF16;
    default: TORCH_CHECK(false, "sparse_mlp: unsupported dtype ", t, " (float32, float16, bfloat16)");
  }
  return -1;
}

static void* cur_stream(const c10::Device& d) {
  return static_cast<void*>(c10::cuda::getCurrentCUDAStream(d.index()).stream());
}

class WeightCache : public torch::CustomClassHolder {
 public:
  // WeightCache::WeightCache (weight_cache.h:148-153)
  WeightCache(const torch::Tensor& init_mask, int64_t hidden_size, const torch::Tensor& gate_weight,
              const torch::Tensor& up_weight, const torch::Tensor& down_weight, bool has_gate) {
    TORCH_CHECK(up_weight.defined() && up_weight.is_cuda(),
                "WeightCache: weights must be CUDA tensors (this build has no CPU path)");
    TORCH_CHECK(up_weight.dim() == 2 && down_weight.dim() == 2, "WeightCache: up/down weights must be 2-D");
    device_ = up_weight.device();
    dtype_ = up_weight.scalar_type();
    has_gate_ = has_gate;
    H_ = hidden_size;
    I_ = up_weight.size(0);
    TORCH_CHECK(up_weight.size(1) == H_, "WeightCache: up_weight must be [intermediate, hidden]");
    TORCH_CHECK(down_weight.size(0) == H_ && down_weight.size(1) == I_, "WeightCache: down_weight must be [hidden, intermediate]");
    c10::cuda::CUDAGuard guard(device_);
    auto up = up_weight.contiguous();
    auto down = down_weight.to(device_, dtype_).contiguous();
    torch::Tensor gate;
    if (has_gate) {
      TORCH_CHECK(gate_weight.defined() && gate_weight.dim() == 2 && gate_weight.size(0) == I_ && gate_weight.size(1) == H_,
                  "WeightCache: gate_weight must be [intermediate, hidden]");
      gate = gate_weight.to(device_, dtype_).contiguous();
    }
    auto mask = init_mask.to(device_, torch::kBool).contiguous();
    TORCH_CHECK(mask.numel() == I_, "WeightCache: init_mask must have intermediate_size elements");
    check(stx_cache_create(&c_, I_, H_, to_stx_dtype(dtype_), has_gate ? 1 : 0, has_gate ? gate.data_ptr() : nullptr,
                           up.data_ptr(), down.data_ptr(), static_cast<const uint8_t*>(mask.data_ptr()), 0,
                           cur_stream(device_)),
          "WeightCache");
    // the temporaries above are consumed by work enqueued on the current stream
    c10::cuda::getCurrentCUDAStream(device_.index()).synchronize();
  }
  ~WeightCache() override { stx_cache_destroy(c_); }

  // WeightCache::update_active_weights (weight_cache.h:229-359)
  void update_active_weights(const torch::Tensor& mask) {
    c10::cuda::CUDAGuard guard(device_);
    auto m = mask.to(device_, torch::kBool).contiguous();
    TORCH_CHECK(m.numel() == I_, "update_active_weights: mask must have ", I_, " elements");
    check(stx_cache_update(c_, static_cast<const uint8_t*>(m.data_ptr()), cur_stream(device_)), "update_active_weights");
    if (!mask.is_cuda() || mask.scalar_type() != torch::kBool) {
      // `m` is a temporary copy: keep it alive until the update has consumed it
      c10::cuda::getCurrentCUDAStream(device_.index()).synchronize();
    }
  }

  // WeightCache::get_concat_weight (weight_cache.h:362-366)
  torch::Tensor get_concat_weight() {
    c10::cuda::CUDAGuard guard(device_);
    void* p = nullptr;
    int64_t rows = 0;
    check(stx_cache_concat_weight(c_, &p, &rows, cur_stream(device_)), "get_concat_weight");
    return view(p, {rows, H_}, {H_, 1});
  }

  // WeightCache::get_active_down_weight (weight_cache.h:368-372): [H,K] with strides (1,H)
  torch::Tensor get_active_down_weight() {
    c10::cuda::CUDAGuard guard(device_);
    void* p = nullptr;
    int64_t k = 0;
    check(stx_cache_active_down(c_, &p, &k, cur_stream(device_)), "get_active_down_weight");
    return view(p, {H_, k}, {1, H_});
  }

  // WeightCache::get_num_active (weight_cache.h:374-377; not registered by the reference)
  int64_t get_num_active() {
    c10::cuda::CUDAGuard guard(device_);
    int64_t k = 0;
    const int rc = stx_cache_num_active(c_, &k, cur_stream(device_));
    if (rc == STX_ERR_CACHE_INVALID || rc == STX_ERR_NO_ACTIVE) return k;
    check(rc, "get_num_active");
    return k;
  }

  // The reference's private active_indices (weight_cache.h:44) as an int64 CPU tensor.
  torch::Tensor get_active_indices() {
    c10::cuda::CUDAGuard guard(device_);
    auto out32 = torch::empty({I_}, torch::dtype(torch::kInt32));
    int64_t k = 0;
    check(stx_cache_active_indices(c_, out32.data_ptr<int32_t>(), I_, &k, cur_stream(device_)), "get_active_indices");
    return out32.narrow(0, 0, k).to(torch::kInt64);
  }

  // SkipMLP._forward_sparse_weight_cache (modeling_skip.py:114-117) over this cache without the two
  // getters: K stays on the device, nothing synchronises, so the call can be captured in a CUDA graph.
  // Returns down_proj_buffer (resized to the input's rows like sparse_mlp_op.cpp:107-112 does).
  torch::Tensor sparse_forward(const torch::Tensor& input, torch::Tensor down_proj_buffer, const std::string& activation_fn) {
    TORCH_CHECK(input.is_cuda() && down_proj_buffer.is_cuda(), "WeightCache.sparse_forward: CUDA tensors required");
    TORCH_CHECK(input.scalar_type() == dtype_ && down_proj_buffer.scalar_type() == dtype_,
                "WeightCache.sparse_forward: tensors must have the cache's dtype");
    const int act = stx_act_from_name(activation_fn.c_str());
    TORCH_CHECK(act >= 0, "WeightCache.sparse_forward: unknown activation '", activation_fn, "'");
    c10::cuda::CUDAGuard guard(device_);
    auto shape = input.sizes().vec();
    TORCH_CHECK(!shape.empty() && shape.back() == H_, "WeightCache.sparse_forward: last dimension must be ", H_);
    auto x = input.contiguous().view({-1, H_});
    const int64_t B = x.size(0);
    if (down_proj_buffer.dim() != 2 || down_proj_buffer.size(0) != B || down_proj_buffer.size(1) != H_) down_proj_buffer.resize_({B, H_});
    TORCH_CHECK(down_proj_buffer.is_contiguous(), "WeightCache.sparse_forward: the buffer must be contiguous");
    if (!scratch_.defined() || scratch_rows_ < B) {
      size_t bytes = 0;
      check(stx_mlp_scratch_bytes(B, H_, I_, &bytes), "sparse_forward");
      scratch_ = torch::zeros({static_cast<int64_t>(bytes)}, torch::TensorOptions().dtype(torch::kUInt8).device(device_));
      scratch_rows_ = B;
      scratch_last_ = B;
    } else if (scratch_last_ != B) {  // the zeroed head of the scratch depends on the row count
      scratch_.zero_();
      scratch_last_ = B;
    }
    check(stx_cache_mlp_forward(c_, x.data_ptr(), B, down_proj_buffer.data_ptr(), act, scratch_.data_ptr(), cur_stream(device_)),
          "sparse_forward");
    return shape.size() > 2 ? down_proj_buffer.view(shape) : down_proj_buffer;
  }

  stx_cache_t* handle() const { return c_; }

 private:
  torch::Tensor view(void* p, std::vector<int64_t> sizes, std::vector<int64_t> strides) {
    // The tensor aliases cache-owned memory; it keeps the cache alive.
    auto self = c10::intrusive_ptr<WeightCache>::unsafe_reclaim_from_nonowning(this);
    return torch::from_blob(
        p, sizes, strides, [self](void*) mutable { self.reset(); }, torch::TensorOptions().dtype(dtype_).device(device_));
  }

  stx_cache_t* c_ = nullptr;
  torch::Tensor scratch_;  // of sparse_forward: sized for scratch_rows_ rows, last used with scratch_last_
  int64_t scratch_rows_ = 0, scratch_last_ = 0;
  int64_t H_ = 0, I_ = 0;
  bool has_gate_ = true;
  c10::ScalarType dtype_ = c10::kFloat;
  c10::Device device_ = c10::Device(c10::kCUDA, 0);
};

// Zero-initialised scratch per (device, stream).  A call leaves the leading counter and fp32
// accumulator (256 + 4*B*H bytes, rounded up to 256) zeroed again, but that region's extent
// depends on B and H and the bytes behind it hold activations and partial sums of the last call:
// when a call's (B,H) differs from the previous one on the same buffer, the leading region of the
// new shape is cleared on the stream first.
static void* mlp_scratch(const c10::Device& dev, void* stream, size_t bytes, int64_t B, int64_t H) {
  struct Entry {
    torch::Tensor buf;
    int64_t B = 0, H = 0;
  };
  static std::mutex mu;
  static std::map<std::pair<int, void*>, Entry> cache;
  std::lock_guard<std::mutex> lock(mu);
  Entry& e = cache[std::make_pair(static_cast<int>(dev.index()), stream)];
  if (!e.buf.defined() || static_cast<size_t>(e.buf.numel()) < bytes) {
    e.buf = torch::zeros({static_cast<int64_t>(bytes)}, torch::TensorOptions().dtype(torch::kUInt8).device(dev));
  } else if (e.B != B || e.H != H) {
    const size_t lead = std::min<size_t>(256 + (static_cast<size_t>(B) * H * 4 + 255) / 256 * 256, e.buf.numel());
    const cudaError_t err = cudaMemsetAsync(e.buf.data_ptr(), 0, lead, static_cast<cudaStream_t>(stream));
    TORCH_CHECK(err == cudaSuccess, "sparse_mlp.forward: clearing the scratch buffer failed: ", cudaGetErrorString(err));
  }
  e.B = B;
  e.H = H;
  return e.buf.data_ptr();
}

// sparse_mlp_forward (sparse_mlp_op.cpp:53-76): same positional signature, so the inferred
// schema is forward(Tensor, Tensor, Tensor, Tensor, Tensor, str, bool) -> Tensor.
torch::Tensor sparse_mlp_forward(const torch::Tensor& input, const torch::Tensor& concat_weight,
                                 const torch::Tensor& active_down_weight, torch::Tensor& down_proj_buffer,
                                 torch::Tensor& combined_proj_buffer, const std::string& activation_fn, bool has_gate) {
  TORCH_CHECK(input.is_cuda(), "sparse_mlp.forward: this build runs on CUDA only (input is on ", input.device(), ")");
  TORCH_CHECK(concat_weight.is_cuda() && active_down_weight.is_cuda() && down_proj_buffer.is_cuda() &&
                  combined_proj_buffer.is_cuda(),
              "sparse_mlp.forward: all tensors must be on the input's CUDA device");
  const int act = stx_act_from_name(activation_fn.c_str());
  TORCH_CHECK(act >= 0, "sparse_mlp.forward: unknown activation '", activation_fn, "'");
  const auto dtype = input.scalar_type();
  TORCH_CHECK(concat_weight.scalar_type() == dtype && active_down_weight.scalar_type() == dtype &&
                  down_proj_buffer.scalar_type() == dtype && combined_proj_buffer.scalar_type() == dtype,
              "sparse_mlp.forward: all tensors must share the input dtype");
  c10::cuda::CUDAGuard guard(input.device());

  // flatten to [B,H] (sparse_mlp_op.cpp:88-105)
  auto original_shape = input.sizes().vec();
  const bool needs_reshape = input.dim() > 2;
  const int64_t H = original_shape.back();
  auto x = input.contiguous().view({-1, H});
  const int64_t B = x.size(0);
  const int64_t rows = concat_weight.size(0);
  TORCH_CHECK(concat_weight.dim() == 2 && concat_weight.size(1) == H, "sparse_mlp.forward: concat_weight must be [2K,H]");
  TORCH_CHECK(!has_gate || rows % 2 == 0, "sparse_mlp.forward: gated concat_weight needs an even row count");
  const int64_t K = has_gate ? rows / 2 : rows;
  TORCH_CHECK(active_down_weight.dim() == 2 && active_down_weight.size(0) == H && active_down_weight.size(1) == K,
              "sparse_mlp.forward: active_down_weight must be [H,K]");

  // buffers are resized like the reference does (sparse_mlp_op.cpp:107-117)
  if (down_proj_buffer.dim() != 2 || down_proj_buffer.size(0) != B || down_proj_buffer.size(1) != H)
    down_proj_buffer.resize_({B, H});
  if (combined_proj_buffer.dim() != 2 || combined_proj_buffer.size(0) != B || combined_proj_buffer.size(1) != rows)
    combined_proj_buffer.resize_({B, rows});
  TORCH_CHECK(down_proj_buffer.is_contiguous() && combined_proj_buffer.is_contiguous(),
              "sparse_mlp.forward: buffers must be contiguous");

  auto wcat = concat_weight.contiguous();
  // the kernel wants one contiguous H-row per neuron: that is the storage of a [H,K]
  // tensor with strides (1,H), which is what WeightCache returns
  torch::Tensor wdown = active_down_weight;
  const bool packed = wdown.stride(0) == 1 && (K <= 1 || wdown.stride(1) == H);
  if (!packed) wdown = active_down_weight.t().contiguous().t();

  void* stream = cur_stream(input.device());
  size_t sbytes = 0;
  check(stx_mlp_scratch_bytes(B, H, K, &sbytes), "forward");
  void* scratch = mlp_scratch(input.device(), stream, sbytes, B, H);
  check(stx_sparse_mlp_forward(x.data_ptr(), B, H, wcat.data_ptr(), wdown.data_ptr(), K, down_proj_buffer.data_ptr(),
                               combined_proj_buffer.data_ptr(), act, has_gate ? 1 : 0, to_stx_dtype(dtype), scratch, stream),
        "forward");
  return needs_reshape ? down_proj_buffer.view(original_shape) : down_proj_buffer;
}

// approx_topk_threshold (approx_topk.h:10-87): scores [B,I] -> threshold [B,1]
torch::Tensor approx_topk_threshold(const torch::Tensor& scores, int64_t k) {
  TORCH_CHECK(scores.dim() == 2, "Input scores must be 2D tensor [batch_size, features]");
  TORCH_CHECK(k > 0, "k must be positive");
  TORCH_CHECK(k <= scores.size(1), "k cannot be larger than feature size");
  TORCH_CHECK(scores.is_cuda(), "approx_topk_threshold: this build runs on CUDA only");
  c10::cuda::CUDAGuard guard(scores.device());
  auto s = scores.contiguous();
  const int64_t B = s.size(0), I = s.size(1);
  auto thr = torch::zeros({B, 1}, s.options());
  size_t sbytes = 0;
  check(stx_approx_topk_scratch_bytes(B, I, &sbytes), "approx_topk_threshold");
  auto scratch = torch::empty({static_cast<int64_t>(sbytes)}, torch::TensorOptions().dtype(torch::kUInt8).device(s.device()));
  check(stx_approx_topk_threshold(s.data_ptr(), B, I, k, to_stx_dtype(s.scalar_type()), thr.data_ptr(), scratch.data_ptr(),
                                  cur_stream(s.device())),
        "approx_topk_threshold");
  return thr;
}

// Predictor + rule + batch union in one call (modeling_skip.py:204-214) -> bool [I].
torch::Tensor predict_mask(const torch::Tensor& x, const torch::Tensor& lora_down, const torch::Tensor& lora_up,
                           const std::string& method, double param) {
  TORCH_CHECK(x.is_cuda() && lora_down.is_cuda() && lora_up.is_cuda(), "predict_mask: CUDA tensors required");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t H = x.size(-1);
  auto x2 = x.contiguous().view({-1, H});
  auto A = lora_down.contiguous();
  auto Bm = lora_up.contiguous();
  const int64_t B = x2.size(0), r = A.size(0), I = Bm.size(0);
  TORCH_CHECK(A.size(1) == H && Bm.size(1) == r, "predict_mask: expected down [r,H] and up [I,r]");
  int m = -1;
  if (method == "naive" || method == "threshold") m = STX_MASK_THRESHOLD;
  else if (method == "topk") m = STX_MASK_TOPK;
  else if (method == "statistical_topk") m = STX_MASK_STATISTICAL;
  TORCH_CHECK(m >= 0, "predict_mask: unknown sparsity method '", method, "'");
  size_t sbytes = 0;
  check(stx_predict_scratch_bytes(B, I, r, &sbytes), "predict_mask");
  auto u8 = torch::TensorOptions().dtype(torch::kUInt8).device(x.device());
  auto scratch = torch::empty({static_cast<int64_t>(sbytes)}, u8);
  auto bits = torch::empty({(I + 31) / 32}, torch::TensorOptions().dtype(torch::kInt32).device(x.device()));
  torch::Tensor scores;
  if (m != STX_MASK_THRESHOLD) scores = torch::empty({B, I}, x2.options());
  void* stream = cur_stream(x.device());
  check(stx_predict_mask(x2.data_ptr(), B, H, A.data_ptr(), r, Bm.data_ptr(), I, to_stx_dtype(x2.scalar_type()), m,
                         static_cast<float>(param), static_cast<uint32_t*>(bits.data_ptr()),
                         scores.defined() ? scores.data_ptr() : nullptr, scratch.data_ptr(), stream),
        "predict_mask");
  auto mask = torch::empty({I}, torch::TensorOptions().dtype(torch::kBool).device(x.device()));
  check(stx_mask_bits_to_bytes(static_cast<const uint32_t*>(bits.data_ptr()), I, static_cast<uint8_t*>(mask.data_ptr()), stream),
        "predict_mask");
  return mask;
}

}  // namespace stxb

#ifndef STX_TORCH_NAMESPACE
#define STX_TORCH_NAMESPACE sparse_mlp
#endif

TORCH_LIBRARY(STX_TORCH_NAMESPACE, m) {
  m.class_<stxb::WeightCache>("WeightCache")
      .def(torch::init<const torch::Tensor&, int64_t, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, bool>())
      .def("update_active_weights", &stxb::WeightCache::update_active_weights)
      .def("get_concat_weight", &stxb::WeightCache::get_concat_weight)
      .def("get_active_down_weight", &stxb::WeightCache::get_active_down_weight)
      .def("sparse_forward", &stxb::WeightCache::sparse_forward)
      .def("get_num_active", &stxb::WeightCache::get_num_active)
      .def("get_active_indices", &stxb::WeightCache::get_active_indices);
  m.def("forward", stxb::sparse_mlp_forward);
  m.def("approx_topk_threshold", stxb::approx_topk_threshold);
  m.def("predict_mask", stxb::predict_mask);
}
