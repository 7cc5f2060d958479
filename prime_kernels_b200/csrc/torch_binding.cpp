// torch.ops bindings over the C ABI of libprime_kernels_b200.so.
//
// prime_rmsnorm::fused_rmsnorm_residual keeps the reference schema
// (prime_kernels/rmsnorm/csrc/torch_interface.cpp:65-74): CUDA dispatch key, outputs allocated by
// the op, current stream, errors as TORCH_CHECK.  Shapes are relaxed to any N and C % 32 == 0.
// prime_decode::decode_step exposes the megakernel to the dispatcher (the reference reaches its
// decode kernels through ctypes only; decode_megakernel/__init__.py:72-91).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/all.h>
#include <torch/library.h>

#include <tuple>

#include "../../include/prime_kernels_b200.h"

namespace {

int64_t scale_numel(int64_t N, int64_t C) { return ((N + 127) / 128) * ((C + 127) / 128) * 512; }

void check_rms_inputs(const torch::Tensor& branch, const torch::Tensor& residual, const torch::Tensor& weight) {
    TORCH_CHECK(branch.dim() == 2, "branch must be a 2D (N, C) tensor");
    const int64_t C = branch.size(1);
    TORCH_CHECK(C > 0 && (C % 32) == 0, "C (", C, ") must be a positive multiple of 32");
    TORCH_CHECK(residual.sizes() == branch.sizes(), "residual must have the same shape as branch");
    TORCH_CHECK(weight.dim() == 1 && weight.size(0) == C, "weight must be a 1D (C,) tensor");
    TORCH_CHECK(branch.is_contiguous() && residual.is_contiguous() && weight.is_contiguous(),
                "branch, residual and weight must be contiguous");
    TORCH_CHECK(branch.dtype() == torch::kBFloat16 && residual.dtype() == torch::kBFloat16 &&
                    weight.dtype() == torch::kBFloat16,
                "branch, residual and weight must be bfloat16");
    TORCH_CHECK(branch.is_cuda(), "branch must be a CUDA tensor");
    TORCH_CHECK(residual.device() == branch.device() && weight.device() == branch.device(),
                "all inputs must be on the same device");
}

std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> fused_rmsnorm_residual(const torch::Tensor& branch,
                                                                               const torch::Tensor& residual,
                                                                               const torch::Tensor& weight,
                                                                               double epsilon) {
    check_rms_inputs(branch, residual, weight);
    at::cuda::OptionalCUDAGuard guard{device_of(branch)};
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const int64_t N = branch.size(0), C = branch.size(1);
    auto opts = torch::TensorOptions().device(branch.device());
    torch::Tensor vals = torch::empty({N, C}, opts.dtype(torch::kFloat8_e4m3fn));
    torch::Tensor scales = torch::empty({scale_numel(N, C)}, opts.dtype(torch::kFloat8_e8m0fnu));
    torch::Tensor rrms = torch::empty({N}, opts.dtype(torch::kFloat32));
    const int rc = pk_fused_rmsnorm_residual_forward(vals.data_ptr(), scales.data_ptr(),
                                                     static_cast<float*>(rrms.data_ptr()), branch.const_data_ptr(),
                                                     residual.const_data_ptr(), weight.const_data_ptr(),
                                                     static_cast<float>(epsilon), (int)N, (int)C, stream);
    TORCH_CHECK(rc == 0, "fused_rmsnorm_residual failed: ", pk_status_string(rc));
    return {vals, scales, rrms};
}

std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> fused_rmsnorm_residual_ex(
    const torch::Tensor& branch, const torch::Tensor& residual, const torch::Tensor& weight, double epsilon,
    bool residual_out, bool prenorm_add) {
    check_rms_inputs(branch, residual, weight);
    at::cuda::OptionalCUDAGuard guard{device_of(branch)};
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const int64_t N = branch.size(0), C = branch.size(1);
    auto opts = torch::TensorOptions().device(branch.device());
    torch::Tensor vals = torch::empty({N, C}, opts.dtype(torch::kFloat8_e4m3fn));
    torch::Tensor scales = torch::empty({scale_numel(N, C)}, opts.dtype(torch::kFloat8_e8m0fnu));
    torch::Tensor rrms = torch::empty({N}, opts.dtype(torch::kFloat32));
    torch::Tensor res = residual_out ? torch::empty({N, C}, opts.dtype(torch::kBFloat16))
                                     : torch::empty({0}, opts.dtype(torch::kBFloat16));
    const int rc = pk_fused_rmsnorm_residual_forward_ex(
        vals.data_ptr(), scales.data_ptr(), static_cast<float*>(rrms.data_ptr()),
        residual_out ? res.data_ptr() : nullptr, branch.const_data_ptr(), residual.const_data_ptr(),
        weight.const_data_ptr(), static_cast<float>(epsilon), (int)N, (int)C, prenorm_add ? 1 : 0, stream);
    TORCH_CHECK(rc == 0, "fused_rmsnorm_residual_ex failed: ", pk_status_string(rc));
    return {vals, scales, rrms, res};
}

const void* opt_ptr(const std::optional<torch::Tensor>& t) { return t.has_value() ? t->const_data_ptr() : nullptr; }
void* opt_mptr(const std::optional<torch::Tensor>& t) { return t.has_value() ? t->data_ptr() : nullptr; }

// Returns the status code of the launch (0 = ok); the Python surface turns it into an exception.
int64_t decode_step(const torch::Tensor& input_ids, const torch::Tensor& positions, const torch::Tensor& seq_lens,
                    const torch::Tensor& block_table, const torch::Tensor& slot_mapping, const torch::Tensor& embed,
                    const std::optional<torch::Tensor>& embed_lookup, const torch::Tensor& layers_table,
                    const torch::Tensor& final_norm, const torch::Tensor& kv_table, int64_t k_off, int64_t v_off,
                    int64_t block_stride, int64_t token_stride, int64_t head_stride, int64_t block_size,
                    const torch::Tensor& cos_sin_cache, torch::Tensor out_hidden,
                    std::optional<torch::Tensor> logits, std::optional<torch::Tensor> next_ids,
                    std::optional<torch::Tensor> layer_outputs, torch::Tensor workspace, int64_t hidden,
                    int64_t intermediate, int64_t layers, int64_t q_heads, int64_t kv_heads, int64_t vocab,
                    int64_t weight_format, double eps, int64_t max_seq_len, bool lm_head, bool advance,
                    int64_t path) {
    at::cuda::OptionalCUDAGuard guard{device_of(input_ids)};
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    PkDecodeModel m{(int)hidden, (int)intermediate, (int)layers, (int)q_heads, (int)kv_heads, (int)vocab,
                    (int)weight_format, (float)eps};
    PkDecodeArgs a{};
    a.stream = stream;
    a.batch = (int)input_ids.size(0);
    a.input_ids = input_ids.const_data_ptr();
    a.ids_i64 = input_ids.dtype() == torch::kInt64;
    a.positions = positions.const_data_ptr();
    a.seq_lens = seq_lens.const_data_ptr();
    a.block_table = block_table.const_data_ptr();
    a.bt_stride = (int)block_table.stride(0);
    a.slot_mapping = slot_mapping.const_data_ptr();
    a.layers = layers_table.const_data_ptr();
    a.embed = embed.const_data_ptr();
    a.embed_lookup = opt_ptr(embed_lookup);
    a.final_norm = final_norm.const_data_ptr();
    a.kv_layers = kv_table.const_data_ptr();
    a.k_off = k_off;
    a.v_off = v_off;
    a.block_stride = block_stride;
    a.token_stride = token_stride;
    a.head_stride = head_stride;
    a.block_size = (int)block_size;
    a.cos_sin = cos_sin_cache.const_data_ptr();
    a.cs_fp32 = cos_sin_cache.dtype() == torch::kFloat32;
    a.out_hidden = out_hidden.data_ptr();
    a.logits = opt_mptr(logits);
    a.next_ids = opt_mptr(next_ids);
    a.layer_outputs = opt_mptr(layer_outputs);
    a.workspace = workspace.data_ptr();
    a.workspace_bytes = (size_t)workspace.numel() * workspace.element_size();
    a.max_seq_len = (int)max_seq_len;
    a.lm_head = lm_head;
    a.advance = advance;
    // path 0: chosen by batch size, 1: tensor-core kernel, 2: CUDA-core kernels
    return path == 1 ? pk_decode_step_tc(&m, &a) : (path == 2 ? pk_decode_step_cc(&m, &a) : pk_decode_step(&m, &a));
}

void check_bf16_cuda(const torch::Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.dtype() == torch::kBFloat16, name, " must be a CUDA bfloat16 tensor");
}

std::tuple<torch::Tensor, torch::Tensor> apply_rotary(const torch::Tensor& q, const torch::Tensor& k,
                                                      const torch::Tensor& cos, const torch::Tensor& sin,
                                                      int64_t unsqueeze_dim) {
    check_bf16_cuda(q, "q"); check_bf16_cuda(k, "k"); check_bf16_cuda(cos, "cos"); check_bf16_cuda(sin, "sin");
    TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && cos.dim() == 3 && sin.sizes() == cos.sizes(), "expected 4-D q, k and 3-D cos, sin");
    TORCH_CHECK(unsqueeze_dim == 1 || unsqueeze_dim == 2, "unsqueeze_dim must be 1 or 2");
    TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && cos.is_contiguous() && sin.is_contiguous(), "inputs must be contiguous");
    at::cuda::OptionalCUDAGuard guard{device_of(q)};
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const bool hm = unsqueeze_dim == 1;
    const int64_t B = q.size(0), S = hm ? q.size(2) : q.size(1), D = q.size(3), rot = cos.size(2);
    TORCH_CHECK(cos.size(1) == S && (cos.size(0) == 1 || cos.size(0) == B), "cos must be [1 or B, S, rot]");
    TORCH_CHECK(k.size(0) == B && k.size(3) == D && (hm ? k.size(2) : k.size(1)) == S, "k must match q in batch, seq and head dim");
    torch::Tensor oq = torch::empty_like(q), ok = torch::empty_like(k);
    int rc = pk_apply_rotary(q.const_data_ptr(), oq.data_ptr(), cos.const_data_ptr(), sin.const_data_ptr(), B,
                             (int)(hm ? q.size(1) : q.size(2)), (int)S, (int)D, (int)rot, hm, (int)cos.size(0), stream);
    TORCH_CHECK(rc == 0, "apply_rotary failed: ", pk_status_string(rc));
    rc = pk_apply_rotary(k.const_data_ptr(), ok.data_ptr(), cos.const_data_ptr(), sin.const_data_ptr(), B,
                         (int)(hm ? k.size(1) : k.size(2)), (int)S, (int)D, (int)rot, hm, (int)cos.size(0), stream);
    TORCH_CHECK(rc == 0, "apply_rotary failed: ", pk_status_string(rc));
    return {oq, ok};
}

torch::Tensor rmsnorm_fwd(const torch::Tensor& x, const torch::Tensor& weight, double eps) {
    check_bf16_cuda(x, "x"); check_bf16_cuda(weight, "weight");
    TORCH_CHECK(x.is_contiguous() && weight.dim() == 1 && weight.size(0) == x.size(-1), "x contiguous, weight [H]");
    at::cuda::OptionalCUDAGuard guard{device_of(x)};
    torch::Tensor out = torch::empty_like(x);
    const int64_t H = x.size(-1), rows = x.numel() / H;
    const int rc = pk_rmsnorm_forward(x.const_data_ptr(), nullptr, weight.const_data_ptr(), out.data_ptr(), nullptr, rows,
                                      (int)H, (float)eps, at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(rc == 0, "rmsnorm failed: ", pk_status_string(rc));
    return out;
}

std::tuple<torch::Tensor, torch::Tensor> residual_rmsnorm_fwd(const torch::Tensor& branch, const torch::Tensor& residual,
                                                              const torch::Tensor& weight, double eps) {
    check_bf16_cuda(branch, "branch"); check_bf16_cuda(residual, "residual"); check_bf16_cuda(weight, "weight");
    TORCH_CHECK(branch.is_contiguous() && residual.is_contiguous() && residual.sizes() == branch.sizes(), "branch and residual must be contiguous and match");
    TORCH_CHECK(weight.dim() == 1 && weight.size(0) == branch.size(-1), "weight must be [H]");
    at::cuda::OptionalCUDAGuard guard{device_of(branch)};
    torch::Tensor out = torch::empty_like(branch), sum = torch::empty_like(branch);
    const int64_t H = branch.size(-1), rows = branch.numel() / H;
    const int rc = pk_rmsnorm_forward(branch.const_data_ptr(), residual.const_data_ptr(), weight.const_data_ptr(),
                                      out.data_ptr(), sum.data_ptr(), rows, (int)H, (float)eps, at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(rc == 0, "residual_rmsnorm failed: ", pk_status_string(rc));
    return {out, sum};
}

torch::Tensor swiglu_fwd(const torch::Tensor& gate, const torch::Tensor& up) {
    check_bf16_cuda(gate, "gate"); check_bf16_cuda(up, "up");
    TORCH_CHECK(gate.sizes() == up.sizes() && gate.dim() >= 1 && gate.stride(-1) == 1 && up.stride(-1) == 1, "gate and up must match, contiguous last dim");
    at::cuda::OptionalCUDAGuard guard{device_of(gate)};
    const int64_t cols = gate.size(-1);
    // leading dims may be a strided view of a larger tensor: flatten to rows with one row stride
    torch::Tensor g2 = gate.dim() == 2 ? gate : gate.reshape({-1, cols});
    torch::Tensor u2 = up.dim() == 2 ? up : up.reshape({-1, cols});
    torch::Tensor out = torch::empty(gate.sizes(), gate.options());
    const int rc = pk_swiglu_forward(g2.const_data_ptr(), u2.const_data_ptr(), out.data_ptr(), g2.size(0), (int)cols,
                                     g2.stride(0), u2.stride(0), at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(rc == 0, "swiglu failed: ", pk_status_string(rc));
    return out;
}

std::tuple<torch::Tensor, torch::Tensor> apply_rotary_bwd(const torch::Tensor& gq, const torch::Tensor& gk,
                                                          const torch::Tensor& cos, const torch::Tensor& sin,
                                                          int64_t unsqueeze_dim) {
    check_bf16_cuda(gq, "grad_q"); check_bf16_cuda(gk, "grad_k"); check_bf16_cuda(cos, "cos"); check_bf16_cuda(sin, "sin");
    TORCH_CHECK(gq.dim() == 4 && gk.dim() == 4 && cos.dim() == 3 && sin.sizes() == cos.sizes(), "expected 4-D grads and 3-D cos, sin");
    TORCH_CHECK(unsqueeze_dim == 1 || unsqueeze_dim == 2, "unsqueeze_dim must be 1 or 2");
    TORCH_CHECK(gq.is_contiguous() && gk.is_contiguous() && cos.is_contiguous() && sin.is_contiguous(), "inputs must be contiguous");
    at::cuda::OptionalCUDAGuard guard{device_of(gq)};
    cudaStream_t stream = at::cuda::getCurrentCUDAStream();
    const bool hm = unsqueeze_dim == 1;
    const int64_t B = gq.size(0), S = hm ? gq.size(2) : gq.size(1), D = gq.size(3), rot = cos.size(2);
    TORCH_CHECK(cos.size(1) == S && (cos.size(0) == 1 || cos.size(0) == B), "cos must be [1 or B, S, rot]");
    torch::Tensor dq = torch::empty_like(gq), dk = torch::empty_like(gk);
    int rc = pk_apply_rotary_backward(gq.const_data_ptr(), dq.data_ptr(), cos.const_data_ptr(), sin.const_data_ptr(), B,
                                      (int)(hm ? gq.size(1) : gq.size(2)), (int)S, (int)D, (int)rot, hm, (int)cos.size(0), stream);
    TORCH_CHECK(rc == 0, "apply_rotary backward failed: ", pk_status_string(rc));
    rc = pk_apply_rotary_backward(gk.const_data_ptr(), dk.data_ptr(), cos.const_data_ptr(), sin.const_data_ptr(), B,
                                  (int)(hm ? gk.size(1) : gk.size(2)), (int)S, (int)D, (int)rot, hm, (int)cos.size(0), stream);
    TORCH_CHECK(rc == 0, "apply_rotary backward failed: ", pk_status_string(rc));
    return {dq, dk};
}

// grad_sum is optional (plain rmsnorm, or nothing flowed back through the returned sum)
std::tuple<torch::Tensor, torch::Tensor> rmsnorm_bwd(const torch::Tensor& grad_out, const std::optional<torch::Tensor>& grad_sum,
                                                     const torch::Tensor& x, const torch::Tensor& weight, double eps) {
    check_bf16_cuda(grad_out, "grad_out"); check_bf16_cuda(x, "x"); check_bf16_cuda(weight, "weight");
    TORCH_CHECK(grad_out.is_contiguous() && x.is_contiguous() && grad_out.sizes() == x.sizes(), "grad_out and x must be contiguous and match");
    TORCH_CHECK(weight.dim() == 1 && weight.size(0) == x.size(-1), "weight must be [H]");
    if (grad_sum.has_value()) {
        check_bf16_cuda(*grad_sum, "grad_sum");
        TORCH_CHECK(grad_sum->is_contiguous() && grad_sum->sizes() == x.sizes(), "grad_sum must be contiguous and match x");
    }
    at::cuda::OptionalCUDAGuard guard{device_of(x)};
    const int64_t H = x.size(-1), rows = x.numel() / H;
    torch::Tensor dx = torch::empty_like(x), dw = torch::empty_like(weight);
    torch::Tensor parts = torch::empty({pk_rmsnorm_backward_parts(rows), H}, x.options().dtype(torch::kFloat32));
    const int rc = pk_rmsnorm_backward(grad_out.const_data_ptr(), opt_ptr(grad_sum), x.const_data_ptr(), weight.const_data_ptr(),
                                       dx.data_ptr(), dw.data_ptr(), parts.data_ptr(), rows, (int)H, (float)eps,
                                       at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(rc == 0, "rmsnorm backward failed: ", pk_status_string(rc));
    return {dx, dw};
}

std::tuple<torch::Tensor, torch::Tensor> swiglu_bwd(const torch::Tensor& grad, const torch::Tensor& gate, const torch::Tensor& up) {
    check_bf16_cuda(grad, "grad"); check_bf16_cuda(gate, "gate"); check_bf16_cuda(up, "up");
    TORCH_CHECK(gate.sizes() == up.sizes() && grad.sizes() == gate.sizes() && gate.stride(-1) == 1 && up.stride(-1) == 1,
                "grad, gate and up must match, contiguous last dim");
    at::cuda::OptionalCUDAGuard guard{device_of(gate)};
    const int64_t cols = gate.size(-1);
    torch::Tensor g2 = gate.dim() == 2 ? gate : gate.reshape({-1, cols});
    torch::Tensor u2 = up.dim() == 2 ? up : up.reshape({-1, cols});
    torch::Tensor gr = grad.contiguous();
    torch::Tensor d_gate = torch::empty(gate.sizes(), gate.options()), d_up = torch::empty(gate.sizes(), gate.options());
    const int rc = pk_swiglu_backward(gr.const_data_ptr(), g2.const_data_ptr(), u2.const_data_ptr(), d_gate.data_ptr(),
                                      d_up.data_ptr(), g2.size(0), (int)cols, g2.stride(0), u2.stride(0),
                                      at::cuda::getCurrentCUDAStream());
    TORCH_CHECK(rc == 0, "swiglu backward failed: ", pk_status_string(rc));
    return {d_gate, d_up};
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(prime_elementwise, m) {
    m.def("apply_rotary(Tensor q, Tensor k, Tensor cos, Tensor sin, int unsqueeze_dim) -> (Tensor, Tensor)");
    m.impl("apply_rotary", torch::kCUDA, &apply_rotary);
    m.def("rmsnorm(Tensor x, Tensor weight, float eps) -> Tensor");
    m.impl("rmsnorm", torch::kCUDA, &rmsnorm_fwd);
    m.def("residual_rmsnorm(Tensor branch, Tensor residual, Tensor weight, float eps) -> (Tensor, Tensor)");
    m.impl("residual_rmsnorm", torch::kCUDA, &residual_rmsnorm_fwd);
    m.def("swiglu(Tensor gate, Tensor up) -> Tensor");
    m.impl("swiglu", torch::kCUDA, &swiglu_fwd);
    m.def("apply_rotary_backward(Tensor grad_q, Tensor grad_k, Tensor cos, Tensor sin, int unsqueeze_dim) -> (Tensor, Tensor)");
    m.impl("apply_rotary_backward", torch::kCUDA, &apply_rotary_bwd);
    m.def("rmsnorm_backward(Tensor grad_out, Tensor? grad_sum, Tensor x, Tensor weight, float eps) -> (Tensor, Tensor)");
    m.impl("rmsnorm_backward", torch::kCUDA, &rmsnorm_bwd);
    m.def("swiglu_backward(Tensor grad, Tensor gate, Tensor up) -> (Tensor, Tensor)");
    m.impl("swiglu_backward", torch::kCUDA, &swiglu_bwd);
}

TORCH_LIBRARY_FRAGMENT(prime_rmsnorm, m) {
    m.def("fused_rmsnorm_residual(Tensor branch, Tensor residual, Tensor weight, float epsilon) -> (Tensor, Tensor, Tensor)");
    m.impl("fused_rmsnorm_residual", torch::kCUDA, &fused_rmsnorm_residual);
    m.def("fused_rmsnorm_residual_ex(Tensor branch, Tensor residual, Tensor weight, float epsilon, bool residual_out, "
          "bool prenorm_add) -> (Tensor, Tensor, Tensor, Tensor)");
    m.impl("fused_rmsnorm_residual_ex", torch::kCUDA, &fused_rmsnorm_residual_ex);
}

TORCH_LIBRARY_FRAGMENT(prime_decode, m) {
    // with advance=true the kernel rewrites input_ids, positions, seq_lens and slot_mapping for the next step, and
    // every step appends to the KV caches behind kv_table: all of them are declared mutable
    m.def("decode_step(Tensor(f!) input_ids, Tensor(g!) positions, Tensor(h!) seq_lens, Tensor block_table, "
          "Tensor(i!) slot_mapping, "
          "Tensor embed, Tensor? embed_lookup, Tensor layers_table, Tensor final_norm, Tensor(j!) kv_table, int k_off, "
          "int v_off, int block_stride, int token_stride, int head_stride, int block_size, Tensor cos_sin_cache, "
          "Tensor(a!) out_hidden, Tensor(b!)? logits, Tensor(c!)? next_ids, Tensor(d!)? layer_outputs, "
          "Tensor(e!) workspace, int hidden, int intermediate, int layers, int q_heads, int kv_heads, int vocab, "
          "int weight_format, float eps, int max_seq_len, bool lm_head, bool advance, int path=0) -> int");
    m.impl("decode_step", torch::kCUDA, &decode_step);
}
