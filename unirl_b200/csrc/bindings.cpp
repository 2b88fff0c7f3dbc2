// PyTorch bindings of the sm_100a kernels (module unirl_b200._C).  Tensors are validated here; the .cu
// launchers only see raw pointers.  Outputs are allocated with the caching allocator on the current stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <limits>
#include <map>
#include <mutex>
#include <tuple>

#include "ops.h"
#include "runtime.h"

namespace py = pybind11;
using torch::Tensor;

namespace {

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int dt(const Tensor& t) {
  if (t.scalar_type() == at::kBFloat16) return ub::kBF16;
  if (t.scalar_type() == at::kFloat) return ub::kF32;
  TORCH_CHECK(false, "unirl_b200: unsupported dtype ", t.scalar_type(), " (expected bfloat16 or float32)");
}
void chk(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
const void* optr(const c10::optional<Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

// One device-side status word per GPU: kernels whose bounded waits run out record a code there and drain; the host reads it at
// step boundaries (gemm_status).  The word lives on the device that launches the kernel.
Tensor& gemm_status_tensor() {
  static std::mutex mu;
  static std::map<int, Tensor> per_device;
  const int dev = (int)c10::cuda::current_device();
  std::lock_guard<std::mutex> lock(mu);
  auto it = per_device.find(dev);
  if (it == per_device.end())
    it = per_device.emplace(dev, torch::zeros({1}, torch::dtype(torch::kInt32).device(torch::kCUDA, dev))).first;
  return it->second;
}

// ---------------------------------------------------------------------------------------------- norms
std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const Tensor& w, double eps) {
  chk(x, "x"); chk(w, "weight");
  TORCH_CHECK(x.dim() == 2 && w.numel() == x.size(1) && w.scalar_type() == x.scalar_type(), "rmsnorm: shape/dtype mismatch");
  c10::cuda::CUDAGuard g(x.device());
  auto y = torch::empty_like(x);
  auto rstd = torch::empty({x.size(0)}, x.options().dtype(torch::kFloat));
  ub::rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), x.size(0), (int)x.size(1), (float)eps, dt(x), stream());
  return {y, rstd};
}
std::vector<Tensor> rmsnorm_bwd(const Tensor& gy, const Tensor& x, const Tensor& w, const Tensor& rstd) {
  chk(gy, "gy"); chk(x, "x");
  c10::cuda::CUDAGuard g(x.device());
  auto gx = torch::empty_like(x);
  auto gw = torch::zeros({x.size(1)}, x.options().dtype(torch::kFloat));
  ub::rmsnorm_bwd(gy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), gx.data_ptr(), gw.data_ptr<float>(), x.size(0), (int)x.size(1), dt(x), stream());
  return {gx, gw};
}
std::vector<Tensor> add_rmsnorm_fwd(const Tensor& x, const Tensor& res, const Tensor& w, double eps) {
  chk(x, "x"); chk(res, "residual");
  TORCH_CHECK(x.sizes() == res.sizes() && x.scalar_type() == res.scalar_type(), "add_rmsnorm: mismatch");
  c10::cuda::CUDAGuard g(x.device());
  auto x2 = x.reshape({-1, x.size(-1)});
  auto y = torch::empty_like(x), r = torch::empty_like(x);
  ub::add_rmsnorm_fwd(x.data_ptr(), res.data_ptr(), w.data_ptr(), y.data_ptr(), r.data_ptr(), x2.size(0), (int)x2.size(1), (float)eps, dt(x), stream());
  return {y, r};
}
Tensor layernorm_modulate_fwd(const Tensor& x, const Tensor& shift, const Tensor& scale, double eps) {
  chk(x, "x"); chk(shift, "shift"); chk(scale, "scale");
  TORCH_CHECK(x.dim() == 3 && shift.dim() == 2 && shift.size(0) == x.size(0) && shift.size(1) == x.size(2), "layernorm_modulate: shapes");
  TORCH_CHECK(shift.scalar_type() == x.scalar_type() && scale.scalar_type() == x.scalar_type(), "layernorm_modulate: dtypes");
  c10::cuda::CUDAGuard g(x.device());
  auto y = torch::empty_like(x);
  ub::layernorm_modulate_fwd(x.data_ptr(), shift.data_ptr(), scale.data_ptr(), y.data_ptr(), x.size(0), (int)x.size(1), (int)x.size(2), (float)eps, dt(x), stream());
  return y;
}

// ---------------------------------------------------------------------------------------------- rope
Tensor inv_freq_table(int64_t head_dim, double theta, const torch::Device& dev) {
  // identical expression to the PyTorch oracle: 1 / theta ** (arange(0, D, 2) / D); cached per (D, theta, device)
  static std::map<std::tuple<int64_t, double, int>, Tensor> cache;
  const auto key = std::make_tuple(head_dim, theta, (int)dev.index());
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  auto idx = torch::arange(0, head_dim, 2, torch::dtype(torch::kFloat).device(dev));
  auto t = torch::reciprocal(torch::pow(torch::scalar_tensor(theta, torch::dtype(torch::kFloat).device(dev)), idx / (double)head_dim)).contiguous();
  cache.emplace(key, t);
  return t;
}
std::vector<Tensor> qk_norm_rope_fwd(const Tensor& qkv, const c10::optional<Tensor>& qw, const c10::optional<Tensor>& kw, const Tensor& pos,
                                     int64_t Hq, int64_t Hkv, int64_t D, double theta, double eps) {
  chk(qkv, "qkv"); chk(pos, "positions");
  TORCH_CHECK(qkv.dim() == 2 && qkv.size(1) == (Hq + 2 * Hkv) * D && pos.scalar_type() == at::kInt && D % 2 == 0 && D <= 256, "qk_norm_rope: shapes");
  c10::cuda::CUDAGuard g(qkv.device());
  const int64_t T = qkv.size(0);
  auto q = torch::empty({T, Hq, D}, qkv.options()), k = torch::empty({T, Hkv, D}, qkv.options()), v = torch::empty({T, Hkv, D}, qkv.options());
  auto rstd = torch::empty({T, Hq + Hkv}, qkv.options().dtype(torch::kFloat));
  auto inv = inv_freq_table(D, theta, qkv.device());
  ub::qk_norm_rope_fwd(qkv.data_ptr(), optr(qw), optr(kw), pos.data_ptr<int>(), inv.data_ptr<float>(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                       rstd.data_ptr<float>(), T, (int)Hq, (int)Hkv, (int)D, (float)eps, dt(qkv), stream());
  return {q, k, v, rstd};
}
std::vector<Tensor> layernorm_modulate_bwd(const Tensor& dy, const Tensor& x, const Tensor& scale, double eps) {
  chk(dy, "dy"); chk(x, "x"); chk(scale, "scale");
  TORCH_CHECK(x.dim() == 3 && dy.sizes() == x.sizes() && scale.dim() == 2 && scale.size(0) == x.size(0) && scale.size(1) == x.size(2), "layernorm_modulate_bwd: shapes");
  TORCH_CHECK(dy.scalar_type() == x.scalar_type() && scale.scalar_type() == x.scalar_type() && dy.device() == x.device() && scale.device() == x.device(),
              "layernorm_modulate_bwd: dtypes / devices");
  c10::cuda::CUDAGuard g(x.device());
  auto dx = torch::empty_like(x);
  auto f32 = x.options().dtype(torch::kFloat);
  auto dshift = torch::zeros({x.size(0), x.size(2)}, f32), dscale = torch::zeros({x.size(0), x.size(2)}, f32);
  const bool ok = ub::layernorm_modulate_bwd(dy.data_ptr(), x.data_ptr(), scale.data_ptr(), dx.data_ptr(), dshift.data_ptr<float>(), dscale.data_ptr<float>(),
                                             x.size(0), (int)x.size(1), (int)x.size(2), (float)eps, dt(x), stream());
  TORCH_CHECK(ok, "layernorm_modulate_bwd: rows of ", x.size(2), " elements are too wide for the kernel");
  return {dx, dshift, dscale};
}
// Decode-loop bookkeeping.  Every state tensor is a (row-)view of the generator's state: first dimension B, unit stride inside a row.
static void chk_rows(const Tensor& t, int64_t B, at::ScalarType ty, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == ty && t.dim() >= 1 && t.size(0) == B && t.stride(t.dim() - 1) == 1, "decode bookkeeping: ", name,
              " must be a CUDA tensor of ", B, " rows with the expected dtype");
}
void decode_record_advance(const Tensor& tok, const Tensor& lp, const Tensor& stop, Tensor& out_tokens, Tensor& out_logp, Tensor& cur_tokens, Tensor& lengths,
                           Tensor& finished, Tensor& positions, Tensor& step_counter) {
  const int64_t B = tok.size(0);
  chk_rows(tok, B, at::kLong, "tok"); chk_rows(lp, B, at::kFloat, "lp"); chk_rows(out_tokens, B, at::kLong, "out_tokens"); chk_rows(out_logp, B, at::kFloat, "out_logp");
  chk_rows(cur_tokens, B, at::kLong, "cur_tokens"); chk_rows(lengths, B, at::kLong, "lengths"); chk_rows(finished, B, at::kBool, "finished");
  chk_rows(positions, B, at::kLong, "positions");
  TORCH_CHECK(tok.is_contiguous() && lp.is_contiguous() && stop.is_cuda() && stop.scalar_type() == at::kLong && stop.is_contiguous() && out_tokens.dim() == 2 &&
                  out_logp.sizes() == out_tokens.sizes() && out_logp.stride(0) == out_tokens.stride(0) && step_counter.scalar_type() == at::kLong,
              "decode_record_advance: argument layout");
  c10::cuda::CUDAGuard g(tok.device());
  ub::decode_record_advance(tok.data_ptr<int64_t>(), lp.data_ptr<float>(), stop.data_ptr<int64_t>(), (int)stop.numel(), out_tokens.data_ptr<int64_t>(),
                            out_logp.data_ptr<float>(), out_tokens.stride(0), cur_tokens.data_ptr<int64_t>(), lengths.data_ptr<int64_t>(),
                            reinterpret_cast<uint8_t*>(finished.data_ptr<bool>()), positions.data_ptr<int64_t>(), step_counter.data_ptr<int64_t>(), (int)B,
                            out_tokens.size(1), stream());
}
void decode_prepare(const Tensor& positions, const Tensor& block_tables, int64_t page_size, const Tensor& rope_offset, Tensor& slots, Tensor& seq_lens, Tensor& rope_pos,
                    const c10::optional<Tensor>& prefix_len, const c10::optional<Tensor>& suffix_lens) {
  const int64_t B = positions.size(0);
  chk_rows(positions, B, at::kLong, "positions"); chk_rows(block_tables, B, at::kInt, "block_tables"); chk_rows(rope_offset, B, at::kLong, "rope_offset");
  chk_rows(slots, B, at::kLong, "slots"); chk_rows(seq_lens, B, at::kInt, "seq_lens"); chk_rows(rope_pos, B, at::kLong, "rope_pos");
  const bool cascade = suffix_lens.has_value() && suffix_lens->defined();
  if (cascade) {
    TORCH_CHECK(prefix_len.has_value() && prefix_len->defined(), "decode_prepare: suffix_lens needs prefix_len");
    chk_rows(*prefix_len, B, at::kInt, "prefix_len"); chk_rows(*suffix_lens, B, at::kInt, "suffix_lens");
  }
  TORCH_CHECK(block_tables.dim() == 2 && page_size > 0, "decode_prepare: block_tables [B, pages]");
  c10::cuda::CUDAGuard g(positions.device());
  ub::decode_prepare(positions.data_ptr<int64_t>(), block_tables.data_ptr<int>(), block_tables.stride(0), (int)page_size, rope_offset.data_ptr<int64_t>(),
                     slots.data_ptr<int64_t>(), seq_lens.data_ptr<int>(), rope_pos.data_ptr<int64_t>(), cascade ? prefix_len->data_ptr<int>() : nullptr,
                     cascade ? suffix_lens->data_ptr<int>() : nullptr, (int)B, stream());
}
// Rotary embedding from per-token tables: x [..., L, H, D] (any leading batch dimensions), cos / sin fp32 [L, D / 2].
Tensor rope_table(const Tensor& x, const Tensor& cos_t, const Tensor& sin_t, bool interleaved, bool backward) {
  chk(x, "x"); chk(cos_t, "cos"); chk(sin_t, "sin");
  TORCH_CHECK(x.dim() >= 3 && cos_t.dim() == 2 && cos_t.sizes() == sin_t.sizes() && cos_t.scalar_type() == at::kFloat && sin_t.scalar_type() == at::kFloat,
              "rope_table: x [..., L, H, D], cos / sin fp32 [L, D / 2]");
  const int64_t D = x.size(-1), H = x.size(-2), L = x.size(-3);
  TORCH_CHECK(D % 2 == 0 && cos_t.size(0) == L && cos_t.size(1) == D / 2, "rope_table: table shape [", cos_t.size(0), ", ", cos_t.size(1), "] does not fit x");
  TORCH_CHECK(cos_t.device() == x.device() && sin_t.device() == x.device(), "rope_table: tensors on different devices");
  c10::cuda::CUDAGuard g(x.device());
  auto y = torch::empty_like(x);
  ub::rope_table(x.data_ptr(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), y.data_ptr(), x.numel() / (H * D), (int)H, (int)D, L, interleaved ? 1 : 0,
                 backward ? -1.f : 1.f, dt(x), stream());
  return y;
}
// Inference variant: QK-norm + RoPE + KV-cache write in one launch.  `dense_kv` keeps the [T, Hkv, D] k / v outputs (prefill needs
// them for the packed attention); decode reads the cache only and skips them.
std::vector<Tensor> qk_norm_rope_cache_fwd(const Tensor& qkv, const Tensor& qw, const Tensor& kw, const Tensor& pos, Tensor& kc, Tensor& vc, const Tensor& slots,
                                           int64_t Hq, int64_t Hkv, int64_t D, double theta, double eps, bool dense_kv) {
  chk(qkv, "qkv"); chk(pos, "positions"); chk(kc, "k_cache"); chk(vc, "v_cache"); chk(slots, "slots");
  TORCH_CHECK(qkv.scalar_type() == at::kBFloat16 && kc.scalar_type() == at::kBFloat16 && qkv.dim() == 2 && qkv.size(1) == (Hq + 2 * Hkv) * D, "qk_norm_rope_cache: bf16 qkv");
  TORCH_CHECK(pos.scalar_type() == at::kInt && slots.scalar_type() == at::kLong && slots.numel() == qkv.size(0) && kc.dim() == 4 && kc.size(1) == Hkv && kc.size(3) == D,
              "qk_norm_rope_cache: int32 positions, int64 slots, cache [pages, Hkv, page, D]");
  c10::cuda::CUDAGuard g(qkv.device());
  const int64_t T = qkv.size(0);
  auto q = torch::empty({T, Hq, D}, qkv.options());
  Tensor k, v;
  if (dense_kv) { k = torch::empty({T, Hkv, D}, qkv.options()); v = torch::empty({T, Hkv, D}, qkv.options()); }
  auto inv = inv_freq_table(D, theta, qkv.device());
  const int rc = ub::qk_norm_rope_cache_fwd(qkv.data_ptr(), qw.data_ptr(), kw.data_ptr(), pos.data_ptr<int>(), inv.data_ptr<float>(), q.data_ptr(),
                                            dense_kv ? k.data_ptr() : nullptr, dense_kv ? v.data_ptr() : nullptr, kc.data_ptr(), vc.data_ptr(), slots.data_ptr<int64_t>(), T,
                                            (int)Hq, (int)Hkv, (int)D, (int)kc.size(2), (float)eps, stream());
  TORCH_CHECK(rc == 0, "qk_norm_rope_cache_fwd: unsupported head_dim or launch failure (code ", rc, ")");
  if (dense_kv) return {q, k, v};
  return {q};
}
std::vector<Tensor> qk_norm_rope_bwd(const Tensor& gq, const Tensor& gk, const Tensor& gv, const Tensor& qkv, const c10::optional<Tensor>& qw,
                                     const c10::optional<Tensor>& kw, const Tensor& pos, const Tensor& rstd, int64_t Hq, int64_t Hkv, int64_t D, double theta) {
  chk(gq, "gq"); chk(gk, "gk"); chk(gv, "gv"); chk(qkv, "qkv");
  c10::cuda::CUDAGuard g(qkv.device());
  auto g_qkv = torch::empty_like(qkv);
  auto f32 = qkv.options().dtype(torch::kFloat);
  auto g_qw = torch::zeros({D}, f32), g_kw = torch::zeros({D}, f32);
  auto inv = inv_freq_table(D, theta, qkv.device());
  const bool has_w = qw.has_value() && qw->defined();
  ub::qk_norm_rope_bwd(gq.data_ptr(), gk.data_ptr(), gv.data_ptr(), qkv.data_ptr(), optr(qw), optr(kw), pos.data_ptr<int>(), inv.data_ptr<float>(),
                       rstd.data_ptr<float>(), g_qkv.data_ptr(), has_w ? g_qw.data_ptr<float>() : nullptr, has_w ? g_kw.data_ptr<float>() : nullptr,
                       qkv.size(0), (int)Hq, (int)Hkv, (int)D, dt(qkv), stream());
  return {g_qkv, g_qw, g_kw};
}

// ---------------------------------------------------------------------------------------------- swiglu / kv
Tensor swiglu_fwd(const Tensor& gu) {
  chk(gu, "gate_up");
  c10::cuda::CUDAGuard g(gu.device());
  auto sizes = gu.sizes().vec();
  const int64_t I = sizes.back() / 2;
  sizes.back() = I;
  auto out = torch::empty(sizes, gu.options());
  ub::swiglu_fwd(gu.data_ptr(), out.data_ptr(), gu.numel() / (2 * I), (int)I, dt(gu), stream());
  return out;
}
Tensor swiglu_bwd(const Tensor& gy, const Tensor& gu) {
  chk(gy, "gy"); chk(gu, "gate_up");
  c10::cuda::CUDAGuard g(gu.device());
  auto out = torch::empty_like(gu);
  const int64_t I = gu.size(-1) / 2;
  ub::swiglu_bwd(gy.data_ptr(), gu.data_ptr(), out.data_ptr(), gu.numel() / (2 * I), (int)I, dt(gu), stream());
  return out;
}
void kv_cache_write(const Tensor& k, const Tensor& v, Tensor& kc, Tensor& vc, const Tensor& slots) {
  chk(k, "k"); chk(v, "v"); chk(kc, "k_cache"); chk(vc, "v_cache"); chk(slots, "slot_mapping");
  TORCH_CHECK(slots.scalar_type() == at::kLong && k.scalar_type() == kc.scalar_type(), "kv_cache_write: dtypes");
  c10::cuda::CUDAGuard g(k.device());
  ub::kv_cache_write(k.data_ptr(), v.data_ptr(), kc.data_ptr(), vc.data_ptr(), slots.data_ptr<int64_t>(), k.size(0), (int)k.size(1), (int)k.size(2),
                     (int)kc.size(2), dt(k), stream());
}

// ---------------------------------------------------------------------------------------------- losses
std::vector<Tensor> policy_loss_fwd(const Tensor& n, const Tensor& o, const Tensor& a, const c10::optional<Tensor>& keep, int64_t kind, double p0, double p1) {
  chk(n, "new_logp"); chk(o, "old_logp"); chk(a, "advantages");
  TORCH_CHECK(n.scalar_type() == at::kFloat && o.scalar_type() == at::kFloat && a.scalar_type() == at::kFloat, "policy_loss: fp32 inputs expected");
  TORCH_CHECK(o.numel() == n.numel() && a.numel() == n.numel(), "policy_loss: new_logp, old_logp and advantages must have the same number of elements (",
              n.numel(), ", ", o.numel(), ", ", a.numel(), "); expand advantages to the token shape first");
  TORCH_CHECK(o.device() == n.device() && a.device() == n.device(), "policy_loss: inputs on different devices");
  if (keep.has_value() && keep->defined())
    TORCH_CHECK(keep->is_cuda() && keep->is_contiguous() && keep->numel() == n.numel() && keep->element_size() == 1 && keep->device() == n.device(),
                "policy_loss: keep mask must be a contiguous 1-byte tensor of the same size on the same device");
  c10::cuda::CUDAGuard g(n.device());
  auto loss = torch::empty_like(n), dloss = torch::empty_like(n);
  auto stats = torch::zeros({8}, n.options());
  stats.index_put_({2}, std::numeric_limits<float>::infinity());
  ub::policy_loss_fwd(n.data_ptr<float>(), o.data_ptr<float>(), a.data_ptr<float>(), (const uint8_t*)optr(keep), loss.data_ptr<float>(),
                      dloss.data_ptr<float>(), stats.data_ptr<float>(), n.numel(), (int)kind, (float)p0, (float)p1, stream());
  return {loss, dloss, stats};
}
Tensor mean_sq_diff_rows(const Tensor& a, const Tensor& b) {
  chk(a, "a"); chk(b, "b");
  TORCH_CHECK(a.dim() == 2 && a.sizes() == b.sizes() && a.scalar_type() == b.scalar_type(), "mean_sq_diff_rows: mismatch");
  c10::cuda::CUDAGuard g(a.device());
  auto out = torch::empty({a.size(0)}, a.options().dtype(torch::kFloat));
  ub::mean_sq_diff_rows(a.data_ptr(), b.data_ptr(), out.data_ptr<float>(), a.size(0), a.size(1), dt(a), stream());
  return out;
}
void logprob_dlogits_inplace(Tensor& z, const Tensor& tgt, const Tensor& lse, const Tensor& gg, double temperature) {
  chk(z, "logits"); chk(tgt, "targets"); chk(lse, "lse"); chk(gg, "grad");
  TORCH_CHECK(z.dim() == 2 && tgt.scalar_type() == at::kInt && lse.scalar_type() == at::kFloat && gg.scalar_type() == at::kFloat, "dlogits: dtypes");
  c10::cuda::CUDAGuard g(z.device());
  ub::logprob_dlogits_inplace(z.data_ptr(), tgt.data_ptr<int>(), lse.data_ptr<float>(), gg.data_ptr<float>(), z.size(0), z.size(1), (float)temperature, dt(z), stream());
}

// ---------------------------------------------------------------------------------------------- sampler / optimiser
// Optional per-row random-stream keys: both [B] int64 on the logits' device, or both absent.
std::pair<const int64_t*, const int64_t*> rng_keys(const c10::optional<Tensor>& rows, const c10::optional<Tensor>& steps, int64_t B, const torch::Device& dev) {
  const bool a = rows.has_value() && rows->defined(), b = steps.has_value() && steps->defined();
  TORCH_CHECK(a == b, "sampler: rng_rows and rng_steps come together");
  if (!a) return {nullptr, nullptr};
  TORCH_CHECK(rows->scalar_type() == at::kLong && steps->scalar_type() == at::kLong && rows->numel() >= B && steps->numel() >= B && rows->is_contiguous() &&
              steps->is_contiguous() && rows->device() == dev && steps->device() == dev, "sampler: rng_rows / rng_steps must be contiguous int64 [B] on the logits' device");
  return {rows->data_ptr<int64_t>(), steps->data_ptr<int64_t>()};
}
std::vector<Tensor> sample_full(const Tensor& logits, double temperature, int64_t seed, int64_t step, const c10::optional<Tensor>& step_tensor,
                                c10::optional<Tensor> tok_out, c10::optional<Tensor> logp_out, const c10::optional<Tensor>& rng_rows,
                                const c10::optional<Tensor>& rng_steps) {
  chk(logits, "logits");
  const auto rk = rng_keys(rng_rows, rng_steps, logits.size(0), logits.device());
  TORCH_CHECK(logits.dim() == 2, "sample: logits must be [B, V]");
  c10::cuda::CUDAGuard g(logits.device());
  Tensor tok = tok_out.has_value() && tok_out->defined() ? *tok_out : torch::empty({logits.size(0)}, logits.options().dtype(torch::kLong));
  Tensor lp = logp_out.has_value() && logp_out->defined() ? *logp_out : torch::empty({logits.size(0)}, logits.options().dtype(torch::kFloat));
  ub::sample_full(logits.data_ptr(), logits.size(0), logits.size(1), (float)temperature, (uint64_t)seed, step,
                  step_tensor.has_value() && step_tensor->defined() ? step_tensor->data_ptr<int64_t>() : nullptr, tok.data_ptr<int64_t>(),
                  lp.data_ptr<float>(), dt(logits), stream(), rk.first, rk.second);
  return {tok, lp};
}
std::vector<Tensor> sample_truncated(const Tensor& logits, double temperature, int64_t top_k, double top_p, int64_t seed, int64_t step,
                                     const c10::optional<Tensor>& step_tensor, c10::optional<Tensor> tok_out, c10::optional<Tensor> logp_out,
                                     const c10::optional<Tensor>& rng_rows, const c10::optional<Tensor>& rng_steps) {
  chk(logits, "logits");
  const auto rk = rng_keys(rng_rows, rng_steps, logits.size(0), logits.device());
  TORCH_CHECK(logits.dim() == 2 && temperature > 0 && logits.size(1) < (int64_t(1) << 18), "sample_truncated: logits [B, V < 2^18], temperature > 0");
  c10::cuda::CUDAGuard g(logits.device());
  Tensor tok = tok_out.has_value() && tok_out->defined() ? *tok_out : torch::empty({logits.size(0)}, logits.options().dtype(torch::kLong));
  Tensor lp = logp_out.has_value() && logp_out->defined() ? *logp_out : torch::empty({logits.size(0)}, logits.options().dtype(torch::kFloat));
  TORCH_CHECK(tok.scalar_type() == at::kLong && lp.scalar_type() == at::kFloat && tok.numel() == logits.size(0) && lp.numel() == logits.size(0) && tok.is_cuda() && lp.is_cuda(),
              "sample_truncated: outputs must be int64 / fp32 [B] on the device");
  ub::sample_truncated(logits.data_ptr(), logits.size(0), logits.size(1), (float)temperature, (int)top_k, (float)top_p, (uint64_t)seed, step,
                       step_tensor.has_value() && step_tensor->defined() ? step_tensor->data_ptr<int64_t>() : nullptr, tok.data_ptr<int64_t>(), lp.data_ptr<float>(),
                       dt(logits), stream(), rk.first, rk.second);
  return {tok, lp};
}
void adamw_step(Tensor& master, const Tensor& grad, Tensor& m, Tensor& v, c10::optional<Tensor> low, c10::optional<Tensor> ema, double lr, double b1,
                double b2, double eps, double wd, int64_t step, double grad_scale, double ema_decay, const c10::optional<Tensor>& gst) {
  chk(master, "master"); chk(grad, "grad"); chk(m, "exp_avg"); chk(v, "exp_avg_sq");
  TORCH_CHECK(master.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat, "adamw: fp32 state expected");
  TORCH_CHECK(grad.numel() == master.numel() && m.numel() == master.numel(), "adamw: size mismatch");
  c10::cuda::CUDAGuard g(master.device());
  const bool has_low = low.has_value() && low->defined(), has_ema = ema.has_value() && ema->defined();
  if (has_low) { chk(*low, "low"); TORCH_CHECK(low->numel() == master.numel(), "adamw: low size"); }
  ub::adamw_step(master.data_ptr<float>(), grad.data_ptr(), dt(grad), m.data_ptr<float>(), v.data_ptr<float>(), has_low ? low->data_ptr() : nullptr,
                 has_low ? dt(*low) : ub::kF32, has_ema ? ema->data_ptr<float>() : nullptr, master.numel(), (float)lr, (float)b1, (float)b2, (float)eps,
                 (float)wd, step, (float)grad_scale, gst.has_value() && gst->defined() ? gst->data_ptr<float>() : nullptr, (float)ema_decay, stream());
}
Tensor sum_squares(const Tensor& x) {
  chk(x, "x");
  c10::cuda::CUDAGuard g(x.device());
  auto out = torch::zeros({}, x.options().dtype(torch::kFloat));
  ub::sum_squares(x.data_ptr(), out.data_ptr<float>(), x.numel(), dt(x), stream());
  return out;
}

// ---------------------------------------------------------------------------------------------- SDE
// `v_uncond`: the unconditional branch of a classifier-free-guidance pass (same shape and dtype as `v`, which is then the conditional
// branch); the guided velocity v_u + guidance (v - v_u) is formed inside the kernel.
static const void* uncond_ptr(const c10::optional<Tensor>& vu, const Tensor& v) {
  if (!vu.has_value() || !vu->defined()) return nullptr;
  TORCH_CHECK(vu->is_cuda() && vu->is_contiguous() && vu->sizes() == v.sizes() && vu->scalar_type() == v.scalar_type() && vu->device() == v.device(),
              "sde step: v_uncond must match noise_pred (shape, dtype, device) and be contiguous");
  return vu->data_ptr();
}
std::vector<Tensor> sde_sample_fwd(const Tensor& v, const Tensor& x, const Tensor& noise, const Tensor& ax, const Tensor& av, const Tensor& sd, int64_t mode,
                                   const c10::optional<Tensor>& v_uncond, double guidance) {
  chk(v, "noise_pred"); chk(x, "sample"); chk(noise, "noise");
  TORCH_CHECK(v.sizes() == x.sizes() && v.scalar_type() == x.scalar_type() && noise.scalar_type() == at::kFloat, "sde_sample: mismatch");
  c10::cuda::CUDAGuard g(v.device());
  const int64_t B = v.size(0), N = v.numel() / B;
  auto f32 = v.options().dtype(torch::kFloat);
  auto prev = torch::empty(v.sizes(), f32), mean = torch::empty(v.sizes(), f32), logp = torch::zeros({B}, f32);
  ub::sde_sample_fwd(v.data_ptr(), x.data_ptr(), noise.data_ptr<float>(), ax.data_ptr<float>(), av.data_ptr<float>(), sd.data_ptr<float>(),
                     prev.data_ptr<float>(), mean.data_ptr<float>(), logp.data_ptr<float>(), B, N, (int)mode, dt(v), stream(), uncond_ptr(v_uncond, v), (float)guidance);
  return {prev, mean, logp};
}
std::vector<Tensor> sde_replay_fwd(const Tensor& v, const Tensor& x, const Tensor& prev, const Tensor& ax, const Tensor& av, const Tensor& sd, int64_t mode,
                                   const c10::optional<Tensor>& v_uncond, double guidance) {
  chk(v, "noise_pred"); chk(x, "sample"); chk(prev, "prev_sample");
  TORCH_CHECK(v.sizes() == x.sizes() && v.scalar_type() == x.scalar_type() && prev.scalar_type() == x.scalar_type(), "sde_replay: mismatch");
  c10::cuda::CUDAGuard g(v.device());
  const int64_t B = v.size(0), N = v.numel() / B;
  auto f32 = v.options().dtype(torch::kFloat);
  auto mean = torch::empty(v.sizes(), f32), logp = torch::zeros({B}, f32);
  ub::sde_replay_fwd(v.data_ptr(), x.data_ptr(), prev.data_ptr(), ax.data_ptr<float>(), av.data_ptr<float>(), sd.data_ptr<float>(), mean.data_ptr<float>(),
                     logp.data_ptr<float>(), B, N, (int)mode, dt(v), stream(), uncond_ptr(v_uncond, v), (float)guidance);
  return {mean, logp};
}
// Returns dL/dv, or {dL/dv_cond, dL/dv_uncond} stacked as [2, ...] when `guided` (the forward formed v_u + guidance (v_c - v_u)).
Tensor sde_replay_bwd(const c10::optional<Tensor>& g_mean, const Tensor& g_logp, const Tensor& mean, const Tensor& prev, const Tensor& av,
                      const Tensor& sd, int64_t mode, bool guided, double guidance) {
  chk(mean, "mean");
  c10::cuda::CUDAGuard g(mean.device());
  auto prev32 = prev.to(torch::kFloat).contiguous();
  const int64_t B = mean.size(0), N = mean.numel() / B;
  std::vector<int64_t> shape = mean.sizes().vec();
  if (guided) shape.insert(shape.begin(), 2);
  auto gv = torch::empty(shape, mean.options());
  Tensor gm;
  if (g_mean.has_value() && g_mean->defined()) gm = g_mean->to(torch::kFloat).contiguous();
  ub::sde_replay_bwd(gm.defined() ? gm.data_ptr<float>() : nullptr, g_logp.data_ptr<float>(), mean.data_ptr<float>(), prev32.data_ptr<float>(),
                     av.data_ptr<float>(), sd.data_ptr<float>(), gv.data_ptr<float>(), B, N, (int)mode, stream(),
                     guided ? gv.data_ptr<float>() + mean.numel() : nullptr, (float)guidance);
  return gv;
}

// ---------------------------------------------------------------------------------------------- GEMM family
Tensor gemm_bf16_tn(const Tensor& a, const Tensor& b, const c10::optional<Tensor>& res, int64_t epilogue) {
  chk(a, "a"); chk(b, "weight");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "gemm: A [M,K] and B [N,K] expected");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "gemm: bf16 operands expected");
  c10::cuda::CUDAGuard g(a.device());
  const int64_t M = a.size(0), K = a.size(1);
  const int64_t N = epilogue == ub::kEpiSwiGLU ? b.size(0) / 2 : b.size(0);
  auto c = torch::empty({M, N}, a.options());
  if (res.has_value() && res->defined()) { chk(*res, "residual"); TORCH_CHECK(res->sizes() == c.sizes(), "gemm: residual shape"); }
  const int rc = ub::gemm_bf16_tn(a.data_ptr(), b.data_ptr(), c.data_ptr(), optr(res), (int)M, (int)N, (int)K, (int)K, (int)K, (int)N, (int)epilogue,
                                  gemm_status_tensor().data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_bf16_tn: unsupported shape or launch failure (code ", rc, ") for M=", M, " N=", N, " K=", K);
  return c;
}
// Projection whose output columns are routed box by box (64 columns): `route` is an int64 CUDA tensor [N / 64, 3] holding per box the destination
// address (0 = the returned local matrix, at the box's own columns), stride | extra << 32, and the statistics slot (-1: none; see ops.h).  Destinations may be peer memory.
// `local_cols`: width of the returned local matrix (0: nothing is returned); local boxes are the LAST local_cols columns of the output.
Tensor gemm_bf16_route(const Tensor& a, const Tensor& b, const c10::optional<Tensor>& bias, const Tensor& route, int64_t rows_per_batch, int64_t local_cols,
                       const c10::optional<Tensor>& rowsq) {
  chk(a, "a"); chk(b, "weight");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "gemm route: A [M,K] and B [N,K] expected");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "gemm route: bf16 operands expected");
  const int64_t M = a.size(0), K = a.size(1), N = b.size(0);
  TORCH_CHECK(N % 64 == 0 && local_cols % 64 == 0 && local_cols >= 0 && local_cols <= N, "gemm route: N and local_cols must be multiples of 64");
  TORCH_CHECK(route.is_cuda() && route.device() == a.device() && route.scalar_type() == at::kLong && route.is_contiguous() && route.numel() == (N / 64) * 3,
              "gemm route: int64 routing table [N / 64, 3] on the operands' device");
  float* sq = nullptr;
  if (rowsq.has_value() && rowsq->defined()) {
    TORCH_CHECK(rowsq->is_cuda() && rowsq->device() == a.device() && rowsq->scalar_type() == at::kFloat && rowsq->is_contiguous() && rowsq->numel() % M == 0,
                "gemm route: rowsq must be a contiguous fp32 CUDA tensor [slots, M]");
    sq = rowsq->data_ptr<float>();
  }
  if (bias.has_value() && bias->defined()) { chk(*bias, "bias"); TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == N, "gemm route: bf16 bias [N]"); }
  c10::cuda::CUDAGuard g(a.device());
  auto c = torch::empty({M, local_cols}, a.options());
  // the kernel addresses a local box as C + column, with C the matrix of ALL columns: shift the base so that column N - local_cols is c's first
  void* cbase = local_cols ? static_cast<void*>(static_cast<at::BFloat16*>(c.data_ptr()) - (N - local_cols)) : nullptr;
  const int rc = ub::gemm_bf16_route(a.data_ptr(), b.data_ptr(), optr(bias), cbase, (int)M, (int)N, (int)K, (int)K, (int)K, (int)(local_cols ? local_cols : 8),
                                     route.data_ptr(), (int)rows_per_batch, sq, gemm_status_tensor().data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_bf16_route: unsupported shape or launch failure (code ", rc, ") for M=", M, " N=", N, " K=", K);
  return c;
}
// C (+)= op(A)·op(B) on the tcgen05 kernel.  a_mn: `a` is stored [K, M] (e.g. dY for dW = dYᵀ·X); b_mn: `b` is stored [K, N] (e.g. W for
// dX = dY·W).  Rows may be strided (stride(1) == 1).  `out`: bf16 [M, N] (overwritten) or fp32 [M, N] (C += with `accumulate`, else C =);
// absent: a new bf16 tensor.
Tensor gemm_bf16(const Tensor& a, const Tensor& b, bool a_mn, bool b_mn, c10::optional<Tensor> out, bool accumulate) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "gemm_bf16: 2-D CUDA operands with unit inner stride");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && a.device() == b.device(), "gemm_bf16: bf16 operands on one device");
  const int64_t M = a_mn ? a.size(1) : a.size(0), K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0), Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "gemm_bf16: contraction extents differ (", K, " vs ", Kb, ")");
  c10::cuda::CUDAGuard g(a.device());
  Tensor c = out.has_value() && out->defined() ? *out : torch::empty({M, N}, a.options());
  TORCH_CHECK(c.is_cuda() && c.device() == a.device() && c.dim() == 2 && c.size(0) == M && c.size(1) == N && c.stride(1) == 1, "gemm_bf16: out must be [M, N] on the operands' device");
  const bool f32 = c.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || c.scalar_type() == at::kBFloat16, "gemm_bf16: out must be bf16 or fp32");
  TORCH_CHECK(f32 || !accumulate, "gemm_bf16: accumulation needs an fp32 out");
  const int rc = ub::gemm_bf16_general(a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)M, (int)N, (int)K, (int)a.stride(0), (int)b.stride(0), (int)c.stride(0),
                                       a_mn ? 1 : 0, b_mn ? 1 : 0, f32 ? 1 : 0, accumulate ? 1 : 0, gemm_status_tensor().data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_bf16: unsupported shape / alignment or launch failure (code ", rc, ") for M=", M, " N=", N, " K=", K);
  return c;
}
// dZ = g/T · (onehot(target) − softmax(h·Wᵀ/T)) for the vocabulary rows `w` (a row chunk starting at `col_offset`), bf16 [M, Vc].
Tensor linear_dlogits(const Tensor& h, const Tensor& w, const Tensor& tgt, const Tensor& lse, const Tensor& gout, double temperature, int64_t col_offset) {
  chk(h, "hidden"); chk(w, "weight"); chk(tgt, "targets"); chk(lse, "lse"); chk(gout, "grad");
  TORCH_CHECK(h.dim() == 2 && w.dim() == 2 && h.size(1) == w.size(1) && h.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16, "linear_dlogits: bf16 [M,K] x [Vc,K]");
  TORCH_CHECK(tgt.scalar_type() == at::kInt && lse.scalar_type() == at::kFloat && gout.scalar_type() == at::kFloat && tgt.numel() == h.size(0) &&
              lse.numel() == h.size(0) && gout.numel() == h.size(0), "linear_dlogits: int32 targets, fp32 lse / grad, one per row");
  c10::cuda::CUDAGuard g(h.device());
  auto dz = torch::empty({h.size(0), w.size(0)}, h.options());
  const int rc = ub::linear_dlogits(h.data_ptr(), w.data_ptr(), dz.data_ptr(), (int)h.size(0), (int)w.size(0), (int)h.size(1), (int)h.size(1), (int)w.size(1), (int)w.size(0),
                                    tgt.data_ptr<int>(), lse.data_ptr<float>(), gout.data_ptr<float>(), (float)temperature, (int)col_offset,
                                    gemm_status_tensor().data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "linear_dlogits: unsupported shape or launch failure (code ", rc, ")");
  return dz;
}
// Decode-sized GEMM: one tile per CTA, K split over a thread-block cluster (see gemm_skinny.cu).  epilogue 0 / 1 (residual) / 2 (SwiGLU).
Tensor gemm_bf16_tn_skinny(const Tensor& a, const Tensor& b, const c10::optional<Tensor>& res, const c10::optional<Tensor>& out, int64_t epilogue) {
  chk(a, "a"); chk(b, "weight");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "gemm: A [M,K] and B [N,K] expected");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "gemm: bf16 operands expected");
  c10::cuda::CUDAGuard g(a.device());
  const int64_t M = a.size(0), K = a.size(1);
  const int64_t N = epilogue == ub::kEpiSwiGLU ? b.size(0) / 2 : b.size(0);
  Tensor c;
  if (out.has_value() && out->defined()) {
    chk(*out, "out");
    TORCH_CHECK(out->scalar_type() == at::kBFloat16 && out->dim() == 2 && out->size(0) == M && out->size(1) == N, "gemm: out shape");
    c = *out;
  } else {
    c = torch::empty({M, N}, a.options());
  }
  const bool has_res = res.has_value() && res->defined();
  if (has_res) { chk(*res, "residual"); TORCH_CHECK(res->sizes() == c.sizes() && epilogue != ub::kEpiSwiGLU, "gemm: residual shape / epilogue"); }
  const int rc = ub::gemm_bf16_tn_skinny(a.data_ptr(), b.data_ptr(), c.data_ptr(), optr(res), (int)M, (int)N, (int)K, (int)K, (int)K, (int)N,
                                         has_res ? ub::kEpiResidual : (int)epilogue, gemm_status_tensor().data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "gemm_bf16_tn_skinny: unsupported shape or launch failure (code ", rc, ") for M=", M, " N=", N, " K=", K);
  return c;
}
std::vector<int64_t> gemm_skinny_plan(int64_t M, int64_t N, int64_t K, bool swiglu) {
  int bn = 0, splits = 0;
  ub::gemm_skinny_plan((int)M, (int)N, (int)K, swiglu, &bn, &splits);
  return {bn, splits};
}
int64_t gemm_status(bool reset) {
  auto& st = gemm_status_tensor();
  const int64_t v = st.item<int>();
  if (reset && v != 0) st.zero_();
  return v;
}
// Host-side write of the current device's status word (tests of the error path; no kernel is made to give up for them).
void set_gemm_status(int64_t code) { gemm_status_tensor().fill_((int)code); }
std::vector<Tensor> linear_logprob_fwd(const Tensor& h, const Tensor& w, const Tensor& tgt, double temperature) {
  chk(h, "hidden"); chk(w, "weight"); chk(tgt, "targets");
  TORCH_CHECK(h.dim() == 2 && w.dim() == 2 && h.size(1) == w.size(1) && tgt.scalar_type() == at::kInt && tgt.numel() == h.size(0), "linear_logprob: shapes");
  TORCH_CHECK(h.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16, "linear_logprob: bf16 operands expected");
  c10::cuda::CUDAGuard g(h.device());
  const int64_t M = h.size(0), V = w.size(0), K = h.size(1);
  const int NT = ub::lse_num_tiles((int)V);
  auto f32 = h.options().dtype(torch::kFloat);
  auto pmax = torch::empty({M, NT}, f32), psum = torch::empty({M, NT}, f32), tl = torch::zeros({M}, f32);
  auto lse = torch::empty({M}, f32), logp = torch::empty({M}, f32);
  const int rc = ub::linear_lse(h.data_ptr(), w.data_ptr(), (int)M, (int)V, (int)K, (int)K, (int)K, tgt.data_ptr<int>(), (float)temperature,
                                pmax.data_ptr<float>(), psum.data_ptr<float>(), tl.data_ptr<float>(), nullptr, nullptr, nullptr, 0, 0, nullptr,
                                lse.data_ptr<float>(), logp.data_ptr<float>(), nullptr, gemm_status_tensor().data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "linear_logprob_fwd: launch failure (code ", rc, ")");
  return {logp, lse};
}
std::vector<Tensor> linear_sample(const Tensor& h, const Tensor& w, double temperature, int64_t seed, int64_t step, const c10::optional<Tensor>& step_tensor,
                                  const c10::optional<Tensor>& rng_rows, const c10::optional<Tensor>& rng_steps) {
  const auto rk = rng_keys(rng_rows, rng_steps, h.size(0), h.device());
  chk(h, "hidden"); chk(w, "weight");
  TORCH_CHECK(h.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && h.size(1) == w.size(1), "linear_sample: bf16 [M,K] x [V,K]");
  c10::cuda::CUDAGuard g(h.device());
  const int64_t M = h.size(0), V = w.size(0), K = h.size(1);
  const int NT = ub::lse_num_tiles((int)V);
  auto f32 = h.options().dtype(torch::kFloat);
  auto pmax = torch::empty({M, NT}, f32), psum = torch::empty({M, NT}, f32), pb = torch::empty({M, NT}, f32), pz = torch::empty({M, NT}, f32);
  auto pi = torch::empty({M, NT}, h.options().dtype(torch::kInt));
  auto tok = torch::empty({M}, h.options().dtype(torch::kLong));
  auto logp = torch::empty({M}, f32);
  const int rc = ub::linear_lse(h.data_ptr(), w.data_ptr(), (int)M, (int)V, (int)K, (int)K, (int)K, nullptr, (float)temperature, pmax.data_ptr<float>(),
                                psum.data_ptr<float>(), nullptr, pb.data_ptr<float>(), pi.data_ptr<int>(), pz.data_ptr<float>(), (uint64_t)seed, step,
                                step_tensor.has_value() && step_tensor->defined() ? step_tensor->data_ptr<int64_t>() : nullptr, nullptr,
                                logp.data_ptr<float>(), tok.data_ptr<int64_t>(), gemm_status_tensor().data_ptr<int>(), stream(), rk.first, rk.second);
  TORCH_CHECK(rc == 0, "linear_sample: launch failure (code ", rc, ")");
  return {tok, logp};
}

// ---------------------------------------------------------------------------------------------- decode attention
int64_t decode_workspace_size(int64_t B, int64_t Hq, int64_t D, int64_t max_kv_len) {
  // upper bound over every split count the heuristic may pick for this batch
  return ub::decode_workspace_floats((int)B, (int)Hq, (int)D, 32);
}
Tensor paged_decode_attention(const Tensor& q, const Tensor& kc, const Tensor& vc, const Tensor& bt, const Tensor& sl, double scale,
                              c10::optional<Tensor> workspace, int64_t max_kv_len) {
  chk(q, "q"); chk(kc, "k_cache"); chk(vc, "v_cache"); chk(bt, "block_tables"); chk(sl, "seq_lens");
  TORCH_CHECK(q.dim() == 3 && kc.dim() == 4 && q.scalar_type() == at::kBFloat16 && kc.scalar_type() == at::kBFloat16, "decode attention: bf16 q [B,Hq,D], cache [P,Hkv,page,D]");
  TORCH_CHECK(bt.scalar_type() == at::kInt && sl.scalar_type() == at::kInt, "decode attention: int32 block_tables / seq_lens");
  TORCH_CHECK(bt.dim() == 2 && bt.size(0) == q.size(0) && sl.numel() == q.size(0), "decode attention: block_tables [B, pages] and seq_lens [B] must match q's batch");
  TORCH_CHECK(vc.sizes() == kc.sizes() && vc.scalar_type() == kc.scalar_type() && kc.size(3) == q.size(2), "decode attention: v_cache must have k_cache's shape and head_dim must match q");
  TORCH_CHECK(kc.device() == q.device() && vc.device() == q.device() && bt.device() == q.device() && sl.device() == q.device(), "decode attention: tensors on different devices");
  if (workspace.has_value() && workspace->defined())
    TORCH_CHECK(workspace->is_cuda() && workspace->device() == q.device() && workspace->scalar_type() == at::kFloat && workspace->is_contiguous(),
                "decode attention: workspace must be a contiguous float32 tensor on q's device");
  c10::cuda::CUDAGuard g(q.device());
  const int B = (int)q.size(0), Hq = (int)q.size(1), D = (int)q.size(2), Hkv = (int)kc.size(1), page = (int)kc.size(2);
  const int kv_hint = max_kv_len > 0 ? (int)max_kv_len : (int)(bt.size(1) * page);
  const int splits = ub::decode_num_splits(B, Hkv, kv_hint);
  const int64_t need = ub::decode_workspace_floats(B, Hq, D, splits);
  Tensor ws = workspace.has_value() && workspace->defined() && workspace->numel() >= need ? *workspace
                                                                                           : torch::empty({need}, q.options().dtype(torch::kFloat));
  auto out = torch::empty_like(q);
  const int rc = ub::paged_decode_attention(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), bt.data_ptr<int>(), sl.data_ptr<int>(), out.data_ptr(),
                                            ws.data_ptr<float>(), B, Hq, Hkv, D, page, (int)bt.size(1), splits, (float)scale, gemm_status_tensor().data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "paged_decode_attention: unsupported configuration or launch failure (code ", rc, ")");
  return out;
}

// Packed-sequence flash attention (tcgen05).  q [T, Hq, D], k / v [T, Hkv, D]: bf16, dense in the last two dimensions, rows may be strided
// (views into a fused qkv buffer); cu_seqlens int32 [B + 1].  Returns {out [T, Hq, D], lse fp32 [Hq, T]}.
std::vector<Tensor> attn_varlen_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& cu, int64_t max_seqlen, bool causal, double scale) {
  (void)max_seqlen;
  TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda() && cu.is_cuda() && q.device() == k.device() && q.device() == v.device() && q.device() == cu.device(),
              "attn_varlen_fwd: CUDA tensors on one device");
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3 && q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16,
              "attn_varlen_fwd: bf16 [T, H, D] tensors");
  TORCH_CHECK(k.sizes() == v.sizes() && q.size(0) == k.size(0) && q.size(2) == k.size(2), "attn_varlen_fwd: q / k / v shapes");
  auto dense = [](const Tensor& t) { return t.stride(2) == 1 && t.stride(1) == t.size(2) && t.stride(0) % 8 == 0; };
  TORCH_CHECK(dense(q) && dense(k) && dense(v), "attn_varlen_fwd: heads and features must be dense, row stride a multiple of 8 elements");
  TORCH_CHECK(cu.scalar_type() == at::kInt && cu.is_contiguous() && cu.numel() >= 2, "attn_varlen_fwd: int32 cu_seqlens [B + 1]");
  c10::cuda::CUDAGuard g(q.device());
  const int T = (int)q.size(0), Hq = (int)q.size(1), D = (int)q.size(2), Hkv = (int)k.size(1), B = (int)cu.numel() - 1;
  auto out = torch::empty({T, Hq, D}, q.options());
  auto lse = torch::empty({Hq, T}, q.options().dtype(torch::kFloat));
  const int rc = ub::flash_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), cu.data_ptr<int>(), out.data_ptr(), lse.data_ptr<float>(), T, B, Hq, Hkv, D,
                                         q.stride(0), k.stride(0), v.stride(0), (int64_t)Hq * D, (float)scale, causal ? 1 : 0,
                                         gemm_status_tensor().data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "attn_varlen_fwd: unsupported configuration or launch failure (code ", rc, "); head_dim must be 64 or 128");
  return {out, lse};
}

// Gradients of attn_varlen_fwd: returns {dq [T, Hq, D], dk [T, Hkv, D], dv [T, Hkv, D]} (bf16, dense).
std::vector<Tensor> attn_varlen_bwd(const Tensor& d_out, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& lse, const Tensor& cu,
                                    int64_t max_seqlen, bool causal, double scale) {
  (void)max_seqlen;
  auto dense = [](const Tensor& t) { return t.dim() == 3 && t.stride(2) == 1 && t.stride(1) == t.size(2) && t.stride(0) % 8 == 0; };
  TORCH_CHECK(q.is_cuda() && dense(q) && dense(k) && dense(v) && dense(out) && dense(d_out), "attn_varlen_bwd: bf16 [T, H, D] tensors, dense heads / features");
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16 &&
              d_out.scalar_type() == at::kBFloat16, "attn_varlen_bwd: bf16 tensors");
  TORCH_CHECK(out.sizes() == q.sizes() && d_out.sizes() == q.sizes() && k.sizes() == v.sizes() && k.size(0) == q.size(0) && k.size(2) == q.size(2), "attn_varlen_bwd: shapes");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.dim() == 2 && lse.size(0) == q.size(1) && lse.size(1) == q.size(0), "attn_varlen_bwd: lse fp32 [Hq, T]");
  TORCH_CHECK(cu.scalar_type() == at::kInt && cu.is_contiguous() && cu.numel() >= 2, "attn_varlen_bwd: int32 cu_seqlens [B + 1]");
  for (const Tensor* t : {&k, &v, &out, &d_out, &lse, &cu}) TORCH_CHECK(t->is_cuda() && t->device() == q.device(), "attn_varlen_bwd: tensors on different devices");
  c10::cuda::CUDAGuard g(q.device());
  const int T = (int)q.size(0), Hq = (int)q.size(1), D = (int)q.size(2), Hkv = (int)k.size(1), B = (int)cu.numel() - 1;
  auto dq = torch::empty({T, Hq, D}, q.options());
  auto dk = torch::zeros({T, Hkv, D}, q.options());  // rows outside every sequence stay zero
  auto dv = torch::zeros({T, Hkv, D}, q.options());
  auto ws = torch::empty({ub::flash_attention_bwd_workspace_floats(T, Hq, D)}, q.options().dtype(torch::kFloat));
  const int rc = ub::flash_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), d_out.data_ptr(), lse.data_ptr<float>(), cu.data_ptr<int>(),
                                         dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ws.data_ptr<float>(), T, B, Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0),
                                         out.stride(0), d_out.stride(0), (float)scale, causal ? 1 : 0, gemm_status_tensor().data_ptr<int>(), stream());
  TORCH_CHECK(rc == 0, "attn_varlen_bwd: unsupported configuration or launch failure (code ", rc, ")");
  return {dq, dk, dv};
}

// ---------------------------------------------------------------------------------------------- peer-memory collectives
// Python owns the symmetric allocations (torch symmetric memory); this object only carries their addresses.
struct PyPeerComm {
  ub::PeerComm c;
  Tensor state;  // int32[8]: [0]=tick [1..2]=ctr [4]=status — keeps the device words alive
  PyPeerComm(std::vector<int64_t> bufs, std::vector<int64_t> flags, int rank, Tensor st, double wait_s) : state(std::move(st)) {
    TORCH_CHECK(bufs.size() == flags.size() && !bufs.empty() && (int)bufs.size() <= ub::kMaxPeers, "PeerComm: 1..8 ranks");
    TORCH_CHECK(state.is_cuda() && state.scalar_type() == at::kInt && state.numel() >= 8 && state.is_contiguous(), "PeerComm: state must be int32[8] on the device");
    for (size_t i = 0; i < bufs.size(); ++i) { c.bufs[i] = bufs[i]; c.flags[i] = flags[i]; }
    c.rank = rank; c.world = (int)bufs.size();
    c.tick = reinterpret_cast<uint32_t*>(state.data_ptr<int>());
    c.ctr = c.tick + 1;
    c.status = state.data_ptr<int>() + 4;
    c.wait_ns = (unsigned long long)(wait_s * 1e9);
  }
  void set_bufs(std::vector<int64_t> bufs) {
    TORCH_CHECK((int)bufs.size() == c.world, "PeerComm.set_bufs: world mismatch");
    for (size_t i = 0; i < bufs.size(); ++i) c.bufs[i] = bufs[i];
  }
  int64_t base() const { return c.bufs[c.rank]; }
  // byte distance of a local tensor from this rank's arena base, in elements of the tensor's dtype
  int64_t offset_of(const Tensor& t) const {
    const int64_t d = (int64_t)reinterpret_cast<uintptr_t>(t.data_ptr()) - base();
    TORCH_CHECK(d >= 0 && d % t.element_size() == 0, "tensor does not live in this communicator's arena");
    return d / t.element_size();
  }
};

void peer_allreduce_residual_rmsnorm(PyPeerComm& pc, const Tensor& part, c10::optional<Tensor> residual, c10::optional<Tensor> w, Tensor& x_out,
                                     c10::optional<Tensor> h_out, double eps) {
  chk(part, "partial"); chk(x_out, "x_out");
  TORCH_CHECK(part.scalar_type() == at::kBFloat16 && part.dim() == 2 && x_out.sizes() == part.sizes(), "peer all-reduce: bf16 [T, H]");
  c10::cuda::CUDAGuard g(part.device());
  const int rc = ub::peer_allreduce_residual_rmsnorm(pc.c, pc.offset_of(part), optr(residual), optr(w), x_out.data_ptr(),
                                                     h_out.has_value() && h_out->defined() ? h_out->data_ptr() : nullptr, part.size(0), (int)part.size(1),
                                                     (float)eps, stream());
  TORCH_CHECK(rc == 0, "peer_allreduce_residual_rmsnorm: unsupported shape or launch failure (code ", rc, ")");
}
// x_out = sum over tensor-parallel ranks of (a · wᵀ) (+ residual), the all-reduce done inside the GEMM epilogue.  `stage` (bf16, 2 * world * slot
// elements) and `flags` (int32, world * 1024, zeroed at start-up) are views into this rank's symmetric arena.
void gemm_skinny_allreduce(PyPeerComm& pc, const Tensor& stage, const Tensor& flags, const Tensor& a, const Tensor& w, c10::optional<Tensor> residual, Tensor& x_out) {
  chk(a, "a"); chk(w, "weight"); chk(x_out, "x_out"); chk(stage, "stage"); chk(flags, "flags");
  TORCH_CHECK(a.dim() == 2 && w.dim() == 2 && a.size(1) == w.size(1) && a.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16, "gemm_skinny_allreduce: bf16 A [M,K], W [N,K]");
  TORCH_CHECK(x_out.scalar_type() == at::kBFloat16 && x_out.dim() == 2 && x_out.size(0) == a.size(0) && x_out.size(1) == w.size(0), "gemm_skinny_allreduce: x_out [M, N] bf16");
  TORCH_CHECK(stage.scalar_type() == at::kBFloat16 && flags.scalar_type() == at::kInt && flags.numel() >= (int64_t)pc.c.world * 1024 && stage.numel() % (2 * pc.c.world) == 0,
              "gemm_skinny_allreduce: stage bf16 [2 * world * slot], flags int32 [world * 1024]");
  if (residual.has_value() && residual->defined()) { chk(*residual, "residual"); TORCH_CHECK(residual->sizes() == x_out.sizes() && residual->scalar_type() == at::kBFloat16, "gemm_skinny_allreduce: residual"); }
  c10::cuda::CUDAGuard g(a.device());
  const int64_t slot = stage.numel() / (2 * pc.c.world);
  const int rc = ub::gemm_skinny_allreduce(pc.c, pc.offset_of(stage) * 2, pc.offset_of(flags) * 4, slot, a.data_ptr(), w.data_ptr(), x_out.data_ptr(), optr(residual),
                                           (int)a.size(0), (int)w.size(0), (int)a.size(1), (int)a.size(1), (int)w.size(1), (int)w.size(0), stream());
  TORCH_CHECK(rc == 0, "gemm_skinny_allreduce: unsupported shape or launch failure (code ", rc, ")");
}
void peer_reduce_scatter_sumsq(PyPeerComm& pc, const Tensor& grad_full, Tensor& out, c10::optional<Tensor> sumsq, double scale) {
  chk(grad_full, "grad"); chk(out, "out");
  TORCH_CHECK(grad_full.scalar_type() == at::kFloat && out.scalar_type() == at::kFloat && grad_full.numel() == out.numel() * pc.c.world, "peer reduce-scatter: fp32, grad = world * out");
  c10::cuda::CUDAGuard g(out.device());
  const int rc = ub::peer_reduce_scatter_sumsq(pc.c, pc.offset_of(grad_full), out.numel(), out.data_ptr<float>(),
                                               sumsq.has_value() && sumsq->defined() ? sumsq->data_ptr<float>() : nullptr, (float)scale, stream());
  TORCH_CHECK(rc == 0, "peer_reduce_scatter_sumsq: unsupported shape or launch failure (code ", rc, ")");
}
void peer_adamw_publish(PyPeerComm& pc, const Tensor& replica_full, Tensor& master, const Tensor& grad, Tensor& m, Tensor& v, c10::optional<Tensor> ema,
                        double lr, double b1, double b2, double eps, double wd, int64_t step, c10::optional<Tensor> clip, double ema_decay) {
  chk(replica_full, "replica"); chk(master, "master"); chk(grad, "grad"); chk(m, "exp_avg"); chk(v, "exp_avg_sq");
  TORCH_CHECK(replica_full.scalar_type() == at::kBFloat16 && master.scalar_type() == at::kFloat && grad.scalar_type() == at::kFloat &&
                  m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat, "peer adamw: bf16 replica, fp32 state");
  TORCH_CHECK(replica_full.numel() == master.numel() * pc.c.world && grad.numel() == master.numel() && m.numel() == master.numel() && v.numel() == master.numel(),
              "peer adamw: size mismatch");
  c10::cuda::CUDAGuard g(master.device());
  const int rc = ub::peer_adamw_publish(pc.c, pc.offset_of(replica_full), master.numel(), master.data_ptr<float>(), grad.data_ptr<float>(), m.data_ptr<float>(),
                                        v.data_ptr<float>(), ema.has_value() && ema->defined() ? ema->data_ptr<float>() : nullptr, (float)lr, (float)b1,
                                        (float)b2, (float)eps, (float)wd, step, clip.has_value() && clip->defined() ? clip->data_ptr<float>() : nullptr,
                                        (float)ema_decay, stream());
  TORCH_CHECK(rc == 0, "peer_adamw_publish: unsupported shape or launch failure (code ", rc, ")");
}
void peer_scatter_copy(const Tensor& table, int64_t n_ops, int64_t max_vecs) {
  chk(table, "table");
  TORCH_CHECK(table.scalar_type() == at::kLong && table.numel() >= n_ops * 6, "scatter_copy: int64 table of 6 words per copy");
  c10::cuda::CUDAGuard g(table.device());
  const int rc = ub::peer_scatter_copy(table.data_ptr(), (int)n_ops, max_vecs, stream());
  TORCH_CHECK(rc == 0, "peer_scatter_copy: launch failure (code ", rc, ")");
}
// Ulysses exchange: `staged` is this rank's tensor inside its symmetric arena (same offset on every rank); returns the permuted pull.
Tensor peer_ulysses_exchange(PyPeerComm& pc, const Tensor& staged, int64_t B, int64_t l, int64_t Hp, int64_t D, int64_t mode) {
  chk(staged, "staged");
  TORCH_CHECK(staged.scalar_type() == at::kBFloat16, "ulysses exchange: bf16 expected");
  const int64_t P = pc.c.world;
  TORCH_CHECK(staged.numel() == B * P * l * Hp * D, "ulysses exchange: staged tensor must hold B * P * l * Hp * D elements");
  c10::cuda::CUDAGuard g(staged.device());
  auto out = mode == 0 ? torch::empty({B, P * l, Hp, D}, staged.options()) : torch::empty({B, l, P * Hp, D}, staged.options());
  const int rc = ub::peer_ulysses_exchange(pc.c, pc.offset_of(staged), out.data_ptr(), (int)B, (int)l, (int)Hp, (int)D, (int)mode, stream());
  TORCH_CHECK(rc == 0, "peer_ulysses_exchange: bad arguments or launch failure (code ", rc, ")");
  return out;
}
void peer_barrier(PyPeerComm& pc) {
  c10::cuda::CUDAGuard g(pc.state.device());
  const int rc = ub::peer_barrier(pc.c, stream());
  TORCH_CHECK(rc == 0, "peer_barrier: launch failure (code ", rc, ")");
}

// Shared-prefix decode attention: groups of `rows` consecutive sequences share the pages listed in prefix_tables.
Tensor paged_decode_attention_cascade(const Tensor& q, const Tensor& kc, const Tensor& vc, const Tensor& prefix_tables, const Tensor& prefix_lens,
                                      const Tensor& suffix_tables, const Tensor& suffix_lens, int64_t rows, double scale, c10::optional<Tensor> workspace,
                                      int64_t max_kv_len) {
  chk(q, "q"); chk(kc, "k_cache"); chk(vc, "v_cache"); chk(prefix_tables, "prefix_tables"); chk(prefix_lens, "prefix_lens"); chk(suffix_tables, "suffix_tables");
  chk(suffix_lens, "suffix_lens");
  TORCH_CHECK(q.dim() == 3 && kc.dim() == 4 && q.scalar_type() == at::kBFloat16 && kc.scalar_type() == at::kBFloat16, "cascade attention: bf16 q [B,Hq,D], cache [P,Hkv,page,D]");
  TORCH_CHECK(prefix_tables.scalar_type() == at::kInt && prefix_lens.scalar_type() == at::kInt && suffix_tables.scalar_type() == at::kInt && suffix_lens.scalar_type() == at::kInt,
              "cascade attention: int32 tables / lengths");
  const int B = (int)q.size(0), Hq = (int)q.size(1), D = (int)q.size(2), Hkv = (int)kc.size(1), page = (int)kc.size(2);
  TORCH_CHECK(rows >= 1 && B % rows == 0 && prefix_tables.size(0) == B / rows && prefix_lens.numel() == B / rows && suffix_tables.size(0) == B && suffix_lens.numel() == B,
              "cascade attention: B / rows prefix entries and B suffix entries expected");
  c10::cuda::CUDAGuard g(q.device());
  const int kv_hint = max_kv_len > 0 ? (int)max_kv_len : (int)(suffix_tables.size(1) * page);
  const int splits = ub::decode_num_splits(B + B / (int)rows, Hkv, kv_hint);
  const int64_t need = ub::decode_cascade_workspace_floats(B, Hq, D, splits);
  Tensor ws = workspace.has_value() && workspace->defined() && workspace->numel() >= need ? *workspace : torch::empty({need}, q.options().dtype(torch::kFloat));
  auto out = torch::empty_like(q);
  const int rc = ub::paged_decode_attention_cascade(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), prefix_tables.data_ptr<int>(), prefix_lens.data_ptr<int>(),
                                                    (int)prefix_tables.size(1), suffix_tables.data_ptr<int>(), suffix_lens.data_ptr<int>(), (int)suffix_tables.size(1),
                                                    out.data_ptr(), ws.data_ptr<float>(), B, (int)rows, Hq, Hkv, D, page, splits, (float)scale, stream());
  TORCH_CHECK(rc == 0, "paged_decode_attention_cascade: unsupported configuration or launch failure (code ", rc, ")");
  return out;
}
int64_t decode_cascade_workspace_size(int64_t B, int64_t rows, int64_t Hq, int64_t Hkv, int64_t D, int64_t max_kv_len) {
  return ub::decode_cascade_workspace_floats((int)B, (int)Hq, (int)D, ub::decode_num_splits((int)(B + B / rows), (int)Hkv, (int)max_kv_len));
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "unirl_b200 native kernels (sm_100a)";
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("add_rmsnorm_fwd", &add_rmsnorm_fwd);
  m.def("layernorm_modulate_fwd", &layernorm_modulate_fwd);
  m.def("layernorm_modulate_bwd", &layernorm_modulate_bwd);
  m.def("qk_norm_rope_fwd", &qk_norm_rope_fwd);
  m.def("qk_norm_rope_bwd", &qk_norm_rope_bwd);
  m.def("qk_norm_rope_cache_fwd", &qk_norm_rope_cache_fwd);
  m.def("rope_table", &rope_table);
  m.def("decode_record_advance", &decode_record_advance);
  m.def("decode_prepare", &decode_prepare);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("kv_cache_write", &kv_cache_write);
  m.def("policy_loss_fwd", &policy_loss_fwd);
  m.def("mean_sq_diff_rows", &mean_sq_diff_rows);
  m.def("logprob_dlogits_inplace", &logprob_dlogits_inplace);
  m.def("sample_full", &sample_full, py::arg("logits"), py::arg("temperature"), py::arg("seed"), py::arg("step"), py::arg("step_tensor") = py::none(),
        py::arg("tok_out") = py::none(), py::arg("logp_out") = py::none(), py::arg("rng_rows") = py::none(), py::arg("rng_steps") = py::none());
  m.def("sample_truncated", &sample_truncated, py::arg("logits"), py::arg("temperature"), py::arg("top_k"), py::arg("top_p"), py::arg("seed"), py::arg("step"),
        py::arg("step_tensor") = py::none(), py::arg("tok_out") = py::none(), py::arg("logp_out") = py::none(), py::arg("rng_rows") = py::none(),
        py::arg("rng_steps") = py::none());
  m.def("adamw_step", &adamw_step);
  m.def("sum_squares", &sum_squares);
  m.def("sde_sample_fwd", &sde_sample_fwd, py::arg("v"), py::arg("x"), py::arg("noise"), py::arg("a_x"), py::arg("a_v"), py::arg("std"), py::arg("mode"),
        py::arg("v_uncond") = py::none(), py::arg("guidance") = 1.0);
  m.def("sde_replay_fwd", &sde_replay_fwd, py::arg("v"), py::arg("x"), py::arg("prev"), py::arg("a_x"), py::arg("a_v"), py::arg("std"), py::arg("mode"),
        py::arg("v_uncond") = py::none(), py::arg("guidance") = 1.0);
  m.def("sde_replay_bwd", &sde_replay_bwd, py::arg("g_mean"), py::arg("g_logp"), py::arg("mean"), py::arg("prev"), py::arg("a_v"), py::arg("std"), py::arg("mode"),
        py::arg("guided") = false, py::arg("guidance") = 1.0);
  m.def("attn_varlen_fwd", &attn_varlen_fwd);
  m.def("attn_varlen_bwd", &attn_varlen_bwd);
  m.def("attn_diag", [](bool backward, bool reset) {  // phase timers of the attention kernels: empty unless built with -DUNIRL_B200_ATTN_DIAG
    unsigned long long t[64];
    const int n = backward ? ub::attention_bwd_diag_read(t, reset) : ub::attention_fwd_diag_read(t, reset);
    TORCH_CHECK(n >= 0, "attn_diag: reading the timer table failed");
    return std::vector<int64_t>(t, t + n);
  });
  m.def("gemm_bf16_tn", &gemm_bf16_tn);
  m.def("gemm_bf16", &gemm_bf16, py::arg("a"), py::arg("b"), py::arg("a_mn") = false, py::arg("b_mn") = false, py::arg("out") = py::none(),
        py::arg("accumulate") = false);
  m.def("gemm_bf16_route", &gemm_bf16_route, py::arg("a"), py::arg("b"), py::arg("bias"), py::arg("route"), py::arg("rows_per_batch"), py::arg("local_cols"),
        py::arg("rowsq") = py::none());
  m.def("linear_dlogits", &linear_dlogits);
  m.def("gemm_bf16_tn_skinny", &gemm_bf16_tn_skinny, py::arg("a"), py::arg("b"), py::arg("res") = py::none(), py::arg("out") = py::none(),
        py::arg("epilogue") = 0);
  m.def("gemm_skinny_plan", &gemm_skinny_plan);
  m.def("set_gemm_skinny_splits", &ub::set_gemm_skinny_splits);
  m.def("set_gemm_skinny_debug", [](const c10::optional<Tensor>& trace, bool skip_a) {
    ub::set_gemm_skinny_debug(trace.has_value() && trace->defined() ? reinterpret_cast<unsigned long long*>(trace->data_ptr<int64_t>()) : nullptr, skip_a ? 1 : 0);
  }, py::arg("trace") = py::none(), py::arg("skip_a") = false);
  m.def("set_pdl", &ub::set_pdl);
  m.def("gemm_status", &gemm_status, py::arg("reset") = true);
  m.def("set_gemm_status", &set_gemm_status);
  m.def("per_device_first_use", [](std::vector<int> devices) {
    // exercises the bookkeeping behind the per-device kernel-attribute caches: which calls in `devices` are first uses
    unsigned char flags[ub::kMaxDevices] = {};
    std::vector<bool> first;
    for (int d : devices) first.push_back(ub::per_device_first_use(flags, ub::kMaxDevices, d));
    return first;
  });
  m.def("set_gemm_tile", &ub::set_gemm_tile);
  m.def("linear_logprob_fwd", &linear_logprob_fwd);
  m.def("linear_sample", &linear_sample, py::arg("hidden"), py::arg("weight"), py::arg("temperature"), py::arg("seed"), py::arg("step"),
        py::arg("step_tensor") = py::none(), py::arg("rng_rows") = py::none(), py::arg("rng_steps") = py::none());
  m.def("decode_workspace_size", &decode_workspace_size);
  m.def("paged_decode_attention", &paged_decode_attention);
  m.def("paged_decode_attention_cascade", &paged_decode_attention_cascade);
  m.def("decode_cascade_workspace_size", &decode_cascade_workspace_size);
  py::class_<PyPeerComm>(m, "PeerComm")
      .def(py::init<std::vector<int64_t>, std::vector<int64_t>, int, Tensor, double>(), py::arg("bufs"), py::arg("flags"), py::arg("rank"), py::arg("state"),
           py::arg("wait_s") = 20.0)
      .def("set_bufs", &PyPeerComm::set_bufs)
      .def("offset_of", &PyPeerComm::offset_of)
      .def_readonly("state", &PyPeerComm::state);
  m.def("peer_allreduce_residual_rmsnorm", &peer_allreduce_residual_rmsnorm);
  m.def("gemm_skinny_allreduce", &gemm_skinny_allreduce);
  m.def("peer_reduce_scatter_sumsq", &peer_reduce_scatter_sumsq);
  m.def("peer_adamw_publish", &peer_adamw_publish);
  m.def("peer_ulysses_exchange", &peer_ulysses_exchange);
  m.def("peer_scatter_copy", &peer_scatter_copy);
  m.def("peer_barrier", &peer_barrier);
  py::class_<ub::BlockAllocator>(m, "BlockAllocator")
      .def(py::init<int64_t>())
      .def("reset", &ub::BlockAllocator::reset)
      .def("allocate", &ub::BlockAllocator::allocate)
      .def("free", &ub::BlockAllocator::free)
      .def_property_readonly("num_free", &ub::BlockAllocator::num_free)
      .def_property_readonly("num_pages", &ub::BlockAllocator::num_pages);
}
