// Thin torch-extension binding over the C ABI of libgnb200.so.
//
// Registers torch.ops.gnb200.fwd / bwd with the schemas of the reference's gnop::fwd / gnop::bwd
// (src/gnnhwc/csrc/custom_gn.cpp:10-16, 44-52, 91-94):
//   fwd(Tensor X, Tensor weight, Tensor bias, int G, float eps, int act) -> (Tensor Y, Tensor means, Tensor rstds)
//   bwd(Tensor dy, Tensor X, Tensor weight, Tensor bias, Tensor means, Tensor rstds, int G, int act)
//       -> (Tensor dX, Tensor dweight, Tensor dbias)
// X / dy / Y / dX are logical (N, C, R) tensors, either with strides (R*C, 1, C), i.e. NHWC storage -
// the only layout the reference's ops accept - or contiguous, i.e. NCHW storage, which goes to the
// native channels-first kernels; results have the storage order of X.
// Differences from the reference, all deliberate: the namespace (so both libraries can live in one
// process), means/rstds are fp32 (fp64 for fp64 tensors), every argument is validated, the
// tensor's device is made current, a third op `bwd_f32` returns the parameter gradients as one packed
// [2, C] tensor in the statistics' dtype (the buffer a data-parallel caller all-reduces), and the ops
// carry explicit schemas with a CUDA implementation (the reference registers catch-all functions, which
// cannot be traced).
#include <ATen/Tensor.h>
#include <ATen/ops/empty.h>
#include <ATen/ops/zeros.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <vector>

#include "../../include/gnb200.h"

namespace {

constexpr int kF64 = 3;  // binding-internal code: double tensors go to the gnb200_*_f64 entry points

int dtype_code(const at::Tensor& t, const char* what) {
  switch (t.scalar_type()) {
    case at::kFloat: return GNB200_F32;
    case at::kHalf: return GNB200_F16;
    case at::kBFloat16: return GNB200_BF16;
    case at::kDouble: return kF64;
    default:
      TORCH_CHECK(false, "gnb200: ", what, " has dtype ", t.scalar_type(),
                  "; supported: float32, float16, bfloat16, float64");
  }
  return -1;
}

// Storage order of a logical (N, C, R) tensor: channels-last (strides (R*C, 1, C), the reference's
// layout, custom_gn.cpp:24,66-67) or channels-first (contiguous).  Anything else is refused.
enum Layout { kNHWC = 0, kNCHW = 1 };
Layout layout_of(const at::Tensor& t, const char* what) {
  TORCH_CHECK(t.device().is_cuda(), "gnb200: ", what, " must be a CUDA tensor (there is no CPU path)");
  TORCH_CHECK(t.dim() == 3, "gnb200: ", what, " must be a rank-3 (N, C, R) view, got rank ", t.dim());
  if (t.permute({0, 2, 1}).is_contiguous()) return kNHWC;
  TORCH_CHECK(t.is_contiguous(), "gnb200: ", what,
              " must be channels-last (strides (R*C, 1, C) for sizes (N, C, R)) or contiguous channels-first; got sizes ",
              t.sizes(), " strides ", t.strides());
  return kNCHW;
}

void check_param(const at::Tensor& p, const at::Tensor& like, int64_t C, const char* what) {
  TORCH_CHECK(p.device() == like.device(), "gnb200: ", what, " is on ", p.device(), " but the input is on ",
              like.device());
  TORCH_CHECK(p.scalar_type() == like.scalar_type(), "gnb200: ", what, " has dtype ", p.scalar_type(),
              " but the input has ", like.scalar_type());
  TORCH_CHECK(p.dim() == 1 && p.size(0) == C && p.is_contiguous(), "gnb200: ", what,
              " must be a contiguous vector of num_channels=", C, " elements, got sizes ", p.sizes());
}

// statistics are fp32 for fp32 / fp16 / bf16 tensors and fp64 for fp64 tensors
at::ScalarType stats_dtype(int dtype) { return dtype == kF64 ? at::kDouble : at::kFloat; }

void check_stats(const at::Tensor& s, const at::Tensor& like, int dtype, int64_t N, int64_t G, const char* what) {
  TORCH_CHECK(s.device() == like.device() && s.scalar_type() == stats_dtype(dtype) && s.is_contiguous() &&
                  s.dim() == 2 && s.size(0) == N && s.size(1) == G,
              "gnb200: ", what, " must be the contiguous (N, G) tensor returned by gnb200::fwd for this input");
}

void check_status(int rc) { TORCH_CHECK(rc == GNB200_OK, gnb200_last_error(), " (status ", rc, ")"); }

// a fresh tensor of X's logical sizes and storage order
at::Tensor empty_like_layout(const at::Tensor& X, Layout layout) {
  const int64_t N = X.size(0), C = X.size(1), R = X.size(2);
  return layout == kNHWC ? at::empty({N, R, C}, X.options()).permute({0, 2, 1}) : at::empty({N, C, R}, X.options());
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> gnb200_fwd_op(const at::Tensor& X, const at::Tensor& weight,
                                                             const at::Tensor& bias, int64_t G, double eps,
                                                             int64_t act) {
  const Layout layout = layout_of(X, "X");
  const int64_t N = X.size(0), C = X.size(1), R = X.size(2);
  const int dtype = dtype_code(X, "X");
  check_param(weight, X, C, "weight");
  check_param(bias, X, C, "bias");
  TORCH_CHECK(G >= 1 && C % G == 0, "gnb200: num_channels ", C, " is not divisible by num_groups ", G);
  TORCH_CHECK(act >= 0 && act <= 4, "gnb200: activation code ", act, " is not in 0..4");
  c10::cuda::CUDAGuard guard(X.device());
  at::Tensor Y = empty_like_layout(X, layout);
  at::Tensor means = at::empty({N, G}, X.options().dtype(stats_dtype(dtype)));
  at::Tensor rstds = at::empty({N, G}, X.options().dtype(stats_dtype(dtype)));
  if (X.numel() == 0) return {Y, means, rstds};
  auto stream = c10::cuda::getCurrentCUDAStream().stream();
  if (dtype == kF64) {
    check_status(gnb200_fwd_f64(X.const_data_ptr<double>(), weight.const_data_ptr<double>(),
                                bias.const_data_ptr<double>(), N, R, C, G, eps, (int)act,
                                layout == kNHWC ? GNB200_LAYOUT_NHWC : GNB200_LAYOUT_NCHW, Y.mutable_data_ptr<double>(),
                                means.mutable_data_ptr<double>(), rstds.mutable_data_ptr<double>(), stream));
    return {Y, means, rstds};
  }
  const size_t ws_bytes = layout == kNHWC ? gnb200_fwd_workspace_bytes(N, R, C, G, dtype)
                                          : gnb200_fwd_nchw_workspace_bytes(N, R, C, G, dtype);
  at::Tensor ws = at::empty({(int64_t)ws_bytes}, X.options().dtype(at::kByte));
  auto fn = layout == kNHWC ? &gnb200_fwd : &gnb200_fwd_nchw;
  check_status(fn(X.const_data_ptr(), weight.const_data_ptr(), bias.const_data_ptr(), N, R, C, G, eps, (int)act, dtype,
                  Y.mutable_data_ptr(), means.mutable_data_ptr<float>(), rstds.mutable_data_ptr<float>(),
                  ws_bytes ? ws.mutable_data_ptr() : nullptr, ws_bytes, stream));
  return {Y, means, rstds};
}

// shared body of bwd / bwd_f32: (dX, packed [dgamma | dbeta], dweight, dbias)
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> bwd_impl(const at::Tensor& dy, const at::Tensor& X,
                                                                    const at::Tensor& weight, const at::Tensor& bias,
                                                                    const at::Tensor& means, const at::Tensor& rstds,
                                                                    int64_t G, int64_t act, bool want_typed,
                                                                    c10::ArrayRef<int64_t> peer_ptrs = {}, int64_t rank = 0) {
  const Layout layout = layout_of(X, "X");
  const int64_t N = X.size(0), C = X.size(1), R = X.size(2);
  const int dtype = dtype_code(X, "X");
  TORCH_CHECK(dy.sizes() == X.sizes() && dy.scalar_type() == X.scalar_type() && dy.device() == X.device(),
              "gnb200: dy must match X in sizes, dtype and device");
  TORCH_CHECK(X.numel() == 0 || layout_of(dy, "dy") == layout || C == 1 || R == 1,
              "gnb200: dy must have the storage order of X; got sizes ", dy.sizes(), " strides ", dy.strides());
  check_param(weight, X, C, "weight");
  check_param(bias, X, C, "bias");
  TORCH_CHECK(G >= 1 && C % G == 0, "gnb200: num_channels ", C, " is not divisible by num_groups ", G);
  TORCH_CHECK(act >= 0 && act <= 4, "gnb200: activation code ", act, " is not in 0..4");
  check_stats(means, X, dtype, N, G, "means");
  check_stats(rstds, X, dtype, N, G, "rstds");
  c10::cuda::CUDAGuard guard(X.device());
  at::Tensor dX = empty_like_layout(X, layout);
  at::Tensor dparam = at::empty({2, C}, X.options().dtype(stats_dtype(dtype)));
  at::Tensor dweight, dbias;
  if (want_typed && dtype != kF64) {
    dweight = at::empty({C}, X.options());
    dbias = at::empty({C}, X.options());
  }
  if (X.numel() == 0) {
    dparam.zero_();
    if (want_typed) {
      dweight = at::zeros({C}, X.options());
      dbias = at::zeros({C}, X.options());
    }
    return {dX, dparam, dweight, dbias};
  }
  auto stream = c10::cuda::getCurrentCUDAStream().stream();
  // data-parallel ranks of one node: the sum over the ranks happens inside the library's kernels,
  // through the ranks' exchange buffers (peer_ptrs[q] = rank q's buffer as mapped into this process)
  const int world = (int)peer_ptrs.size();
  std::vector<const void*> peers(world);
  for (int q = 0; q < world; ++q) peers[q] = reinterpret_cast<const void*>(static_cast<uintptr_t>(peer_ptrs[q]));
  TORCH_CHECK(world == 0 || dtype != kF64, "gnb200: the in-kernel exchange of parameter gradients is for fp32 / fp16 / bf16 tensors");
  if (dtype == kF64) {
    // the packed buffer is the result: its two rows are dgamma and dbeta
    const size_t ws_bytes = gnb200_bwd_f64_workspace_bytes(N, R, C, G);
    at::Tensor ws = at::empty({(int64_t)ws_bytes}, X.options().dtype(at::kByte));
    double* dp = dparam.mutable_data_ptr<double>();
    check_status(gnb200_bwd_f64(dy.const_data_ptr<double>(), X.const_data_ptr<double>(), weight.const_data_ptr<double>(),
                                bias.const_data_ptr<double>(), means.const_data_ptr<double>(),
                                rstds.const_data_ptr<double>(), N, R, C, G, (int)act,
                                layout == kNHWC ? GNB200_LAYOUT_NHWC : GNB200_LAYOUT_NCHW, dX.mutable_data_ptr<double>(),
                                dp, dp + C, ws.mutable_data_ptr(), ws_bytes, stream));
    if (want_typed) {
      dweight = dparam[0];
      dbias = dparam[1];
    }
    return {dX, dparam, dweight, dbias};
  }
  const size_t ws_bytes = layout == kNHWC ? gnb200_bwd_workspace_bytes(N, R, C, G, dtype)
                                          : gnb200_bwd_nchw_workspace_bytes(N, R, C, G, dtype);
  at::Tensor ws = at::empty({(int64_t)ws_bytes}, X.options().dtype(at::kByte));
  void* dw = want_typed ? dweight.mutable_data_ptr() : nullptr;
  void* db = want_typed ? dbias.mutable_data_ptr() : nullptr;
  if (world > 1 && layout == kNHWC) {
    check_status(gnb200_bwd_peer(dy.const_data_ptr(), X.const_data_ptr(), weight.const_data_ptr(), bias.const_data_ptr(),
                                 means.const_data_ptr<float>(), rstds.const_data_ptr<float>(), N, R, C, G, (int)act, dtype,
                                 dX.mutable_data_ptr(), dparam.mutable_data_ptr<float>(), dw, db,
                                 ws_bytes ? ws.mutable_data_ptr() : nullptr, ws_bytes, peers.data(), (int)rank, world, stream));
    return {dX, dparam, dweight, dbias};
  }
  auto fn = layout == kNHWC ? &gnb200_bwd : &gnb200_bwd_nchw;
  check_status(fn(dy.const_data_ptr(), X.const_data_ptr(), weight.const_data_ptr(), bias.const_data_ptr(),
                  means.const_data_ptr<float>(), rstds.const_data_ptr<float>(), N, R, C, G, (int)act, dtype,
                  dX.mutable_data_ptr(), dparam.mutable_data_ptr<float>(), dw, db,
                  ws_bytes ? ws.mutable_data_ptr() : nullptr, ws_bytes, stream));
  if (world > 1)  // channels-first: the exchange follows the backward as a kernel of its own
    check_status(gnb200_allreduce_param_grads(dparam.mutable_data_ptr<float>(), dw, db, C, dtype, peers.data(), (int)rank,
                                              world, stream));
  return {dX, dparam, dweight, dbias};
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

// bwd_f32 with the sum of the parameter gradients over the data-parallel ranks of one node done
// inside the kernels (gnb200_bwd_peer): peer_ptrs[q] is the address of rank q's exchange buffer in
// this process, `rank` this process's index in that list.
std::tuple<at::Tensor, at::Tensor> gnb200_bwd_f32_peer_op(const at::Tensor& dy, const at::Tensor& X,
                                                          const at::Tensor& weight, const at::Tensor& bias,
                                                          const at::Tensor& means, const at::Tensor& rstds, int64_t G,
                                                          int64_t act, c10::ArrayRef<int64_t> peer_ptrs, int64_t rank) {
  TORCH_CHECK(peer_ptrs.size() >= 1 && rank >= 0 && rank < (int64_t)peer_ptrs.size(),
              "gnb200: rank ", rank, " is not an index into the ", peer_ptrs.size(), " exchange buffers");
  auto r = bwd_impl(dy, X, weight, bias, means, rstds, G, act, false, peer_ptrs, rank);
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
  m.def("bwd_f32_peer(Tensor dy, Tensor X, Tensor weight, Tensor bias, Tensor means, Tensor rstds, int G, int act, "
        "int[] peer_ptrs, int rank) -> (Tensor, Tensor)");
}

TORCH_LIBRARY_IMPL(gnb200, CUDA, m) {
  m.impl("fwd", &gnb200_fwd_op);
  m.impl("bwd", &gnb200_bwd_op);
  m.impl("bwd_f32", &gnb200_bwd_f32_op);
  m.impl("bwd_f32_peer", &gnb200_bwd_f32_peer_op);
}

TORCH_LIBRARY_IMPL(gnb200, CPU, m) {
  m.impl("fwd", &gnb200_fwd_op);
  m.impl("bwd", &gnb200_bwd_op);
  m.impl("bwd_f32", &gnb200_bwd_f32_op);
}
