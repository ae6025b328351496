// Thin torch-extension binding over the C ABI of libgnb200.so.
//
// Registers torch.ops.gnb200.fwd / bwd with the schemas of the reference's gnop::fwd / gnop::bwd
// (src/gnnhwc/csrc/custom_gn.cpp:10-16, 44-52, 91-94):
//   fwd(Tensor X, Tensor weight, Tensor bias, int G, float eps, int act) -> (Tensor Y, Tensor means, Tensor rstds)
//   bwd(Tensor dy, Tensor X, Tensor weight, Tensor bias, Tensor means, Tensor rstds, int G, int act)
//       -> (Tensor dX, Tensor dweight, Tensor dbias)
// X / dy / Y / dX are logical (N, C, R) tensors with strides (R*C, 1, C), i.e. NHWC storage.
// Differences from the reference, all deliberate: the namespace (so both libraries can live in one
// process), means/rstds are fp32, every argument is validated, the tensor's device is made current,
// a third op `bwd_f32` returns the parameter gradients as one packed fp32 [2, C] tensor (the
// buffer a data-parallel caller all-reduces), and the ops carry explicit schemas with a CUDA
// implementation (the reference registers catch-all functions, which cannot be traced).
#include <ATen/Tensor.h>
#include <ATen/ops/empty.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include "../../include/gnb200.h"

namespace {

int dtype_code(const at::Tensor& t, const char* what) {
  switch (t.scalar_type()) {
    case at::kFloat: return GNB200_F32;
    case at::kHalf: return GNB200_F16;
    case at::kBFloat16: return GNB200_BF16;
    default:
      TORCH_CHECK(false, "gnb200: ", what, " has dtype ", t.scalar_type(), "; supported: float32, float16, bfloat16");
  }
  return -1;
}

// (N, C, R) view over NHWC storage: the (N, R, C) permutation must be contiguous.
void check_nhwc3(const at::Tensor& t, const char* what) {
  TORCH_CHECK(t.device().is_cuda(), "gnb200: ", what, " must be a CUDA tensor (there is no CPU path)");
  TORCH_CHECK(t.dim() == 3, "gnb200: ", what, " must be a rank-3 (N, C, R) view, got rank ", t.dim());
  TORCH_CHECK(t.permute({0, 2, 1}).is_contiguous(), "gnb200: ", what,
              " must be channels-last: strides (R*C, 1, C) for sizes (N, C, R); got sizes ", t.sizes(), " strides ",
              t.strides());
}

void check_param(const at::Tensor& p, const at::Tensor& like, int64_t C, const char* what) {
  TORCH_CHECK(p.device() == like.device(), "gnb200: ", what, " is on ", p.device(), " but the input is on ",
              like.device());
  TORCH_CHECK(p.scalar_type() == like.scalar_type(), "gnb200: ", what, " has dtype ", p.scalar_type(),
              " but the input has ", like.scalar_type());
  TORCH_CHECK(p.dim() == 1 && p.size(0) == C && p.is_contiguous(), "gnb200: ", what,
              " must be a contiguous vector of num_channels=", C, " elements, got sizes ", p.sizes());
}

void check_stats(const at::Tensor& s, const at::Tensor& like, int64_t N, int64_t G, const char* what) {
  TORCH_CHECK(s.device() == like.device() && s.scalar_type() == at::kFloat && s.is_contiguous() && s.dim() == 2 &&
                  s.size(0) == N && s.size(1) == G,
              "gnb200: ", what, " must be the contiguous float32 (N, G) tensor returned by gnb200::fwd");
}

void check_status(int rc) { TORCH_CHECK(rc == GNB200_OK, gnb200_last_error(), " (status ", rc, ")"); }

std::tuple<at::Tensor, at::Tensor, at::Tensor> gnb200_fwd_op(const at::Tensor& X, const at::Tensor& weight,
                                                             const at::Tensor& bias, int64_t G, double eps,
                                                             int64_t act) {
  check_nhwc3(X, "X");
  const int64_t N = X.size(0), C = X.size(1), R = X.size(2);
  const int dtype = dtype_code(X, "X");
  check_param(weight, X, C, "weight");
  check_param(bias, X, C, "bias");
  TORCH_CHECK(G >= 1 && C % G == 0, "gnb200: num_channels ", C, " is not divisible by num_groups ", G);
  TORCH_CHECK(act >= 0 && act <= 4, "gnb200: activation code ", act, " is not in 0..4");
  c10::cuda::CUDAGuard guard(X.device());
  at::Tensor Y = at::empty({N, R, C}, X.options());
  at::Tensor means = at::empty({N, G}, X.options().dtype(at::kFloat));
  at::Tensor rstds = at::empty({N, G}, X.options().dtype(at::kFloat));
  if (X.numel() > 0) {
    const size_t ws_bytes = gnb200_fwd_workspace_bytes(N, R, C, G, dtype);
    at::Tensor ws = at::empty({(int64_t)ws_bytes}, X.options().dtype(at::kByte));
    check_status(gnb200_fwd(X.const_data_ptr(), weight.const_data_ptr(), bias.const_data_ptr(), N, R, C, G, eps,
                            (int)act, dtype, Y.mutable_data_ptr(), means.mutable_data_ptr<float>(),
                            rstds.mutable_data_ptr<float>(), ws_bytes ? ws.mutable_data_ptr() : nullptr, ws_bytes,
                            c10::cuda::getCurrentCUDAStream().stream()));
  }
  return {Y.permute({0, 2, 1}), means, rstds};
}

// shared body of bwd / bwd_f32
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> bwd_impl(const at::Tensor& dy, const at::Tensor& X,
                                                                    const at::Tensor& weight, const at::Tensor& bias,
                                                                    const at::Tensor& means, const at::Tensor& rstds,
                                                                    int64_t G, int64_t act, bool want_typed) {
  check_nhwc3(X, "X");
  check_nhwc3(dy, "dy");
  const int64_t N = X.size(0), C = X.size(1), R = X.size(2);
  const int dtype = dtype_code(X, "X");
  TORCH_CHECK(dy.sizes() == X.sizes() && dy.scalar_type() == X.scalar_type() && dy.device() == X.device(),
              "gnb200: dy must match X in sizes, dtype and device");
  check_param(weight, X, C, "weight");
  check_param(bias, X, C, "bias");
  TORCH_CHECK(G >= 1 && C % G == 0, "gnb200: num_channels ", C, " is not divisible by num_groups ", G);
  TORCH_CHECK(act >= 0 && act <= 4, "gnb200: activation code ", act, " is not in 0..4");
  check_stats(means, X, N, G, "means");
  check_stats(rstds, X, N, G, "rstds");
  c10::cuda::CUDAGuard guard(X.device());
  at::Tensor dX = at::empty({N, R, C}, X.options());
  at::Tensor dparam = at::empty({2, C}, X.options().dtype(at::kFloat));
  at::Tensor dweight, dbias;
  if (want_typed) {
    dweight = at::empty({C}, X.options());
    dbias = at::empty({C}, X.options());
  }
  if (X.numel() > 0) {
    const size_t ws_bytes = gnb200_bwd_workspace_bytes(N, R, C, G, dtype);
    at::Tensor ws = at::empty({(int64_t)ws_bytes}, X.options().dtype(at::kByte));
    check_status(gnb200_bwd(dy.const_data_ptr(), X.const_data_ptr(), weight.const_data_ptr(), bias.const_data_ptr(),
                            means.const_data_ptr<float>(), rstds.const_data_ptr<float>(), N, R, C, G, (int)act, dtype,
                            dX.mutable_data_ptr(), dparam.mutable_data_ptr<float>(),
                            want_typed ? dweight.mutable_data_ptr() : nullptr,
                            want_typed ? dbias.mutable_data_ptr() : nullptr,
                            ws_bytes ? ws.mutable_data_ptr() : nullptr, ws_bytes,
                            c10::cuda::getCurrentCUDAStream().stream()));
  } else {
    dparam.zero_();
    if (want_typed) {
      dweight.zero_();
      dbias.zero_();
    }
  }
  return {dX.permute({0, 2, 1}), dparam, dweight, dbias};
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> gnb200_bwd_op(const at::Tensor& dy, const at::Tensor& X,
                                                             const at::Tensor& weight, const at::Tensor& bias,
                                                             const at::Tensor& means, const at::Tensor& rstds,
                                                             int64_t G, int64_t act) {
  auto r = bwd_impl(dy, X, weight, bias, means, rstds, G, act, true);
  return {std::get<0>(r), std::get<2>(r), std::get<3>(r)};
}

std::tuple<at::Tensor, at::Tensor> gnb200_bwd_f32_op(const at::Tensor& dy, const at::Tensor& X,
                                                     const at::Tensor& weight, const at::Tensor& bias,
                                                     const at::Tensor& means, const at::Tensor& rstds, int64_t G,
                                                     int64_t act) {
  auto r = bwd_impl(dy, X, weight, bias, means, rstds, G, act, false);
  return {std::get<0>(r), std::get<1>(r)};
}

}  // namespace

// Schemas are declared apart from the implementations so that Python can attach fake-tensor
// kernels and an autograd formula to them (channels_last_groupnorm_b200/_compile.py), which is what
// torch.compile needs.  The CPU registration exists only to fail with the message of check_nhwc3
// instead of the dispatcher's.
TORCH_LIBRARY(gnb200, m) {
  m.def("fwd(Tensor X, Tensor weight, Tensor bias, int G, float eps, int act) -> (Tensor, Tensor, Tensor)");
  m.def("bwd(Tensor dy, Tensor X, Tensor weight, Tensor bias, Tensor means, Tensor rstds, int G, int act) -> "
        "(Tensor, Tensor, Tensor)");
  m.def("bwd_f32(Tensor dy, Tensor X, Tensor weight, Tensor bias, Tensor means, Tensor rstds, int G, int act) -> "
        "(Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(gnb200, CUDA, m) {
  m.impl("fwd", &gnb200_fwd_op);
  m.impl("bwd", &gnb200_bwd_op);
  m.impl("bwd_f32", &gnb200_bwd_f32_op);
}

TORCH_LIBRARY_IMPL(gnb200, CPU, m) {
  m.impl("fwd", &gnb200_fwd_op);
  m.impl("bwd", &gnb200_bwd_op);
  m.impl("bwd_f32", &gnb200_bwd_f32_op);
}
