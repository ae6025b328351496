// Device-side building blocks shared by the forward and backward GroupNorm kernels (sm_100a).
//
// Conventions used throughout:
//   T    element type of the tensors (float, __half, __nv_bfloat16); all arithmetic is fp32
//   VE   elements per thread-vector: 16 bytes worth (4 fp32 / 8 half) on the fast path, 1 on the
//        any-shape fallback
//   a CTA works on a tile of `rows` pixels x CW channels ("column block") of one sample;
//   inside it thread `tid` owns column vector tx = tid % CV and rows ty, ty+TY, ty+2*TY ...
//   (CV = CW / VE, TY = row lanes), so a thread keeps the same channels for its whole loop and
//   consecutive threads touch consecutive 16-byte vectors (coalesced along C).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

namespace gnb200 {

enum : int { kActIdentity = 0, kActRelu = 1, kActSilu = 2, kActGelu = 3, kActGeluTanh = 4 };

constexpr int kMaxThreads = 512;

// ---------------------------------------------------------------------------------------------
// Fixed-order sums
// ---------------------------------------------------------------------------------------------
// Sum over a whole CTA in a fixed order (warp trees, then the warp results in warp order).
// `scratch` holds one float per warp; the total is returned to every thread.
__device__ __forceinline__ float warp_sum(float v);
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nwarps; ++w) t += scratch[w];
  return t;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int delta = 16; delta >= 1; delta >>= 1) v += __shfl_down_sync(0xffffffffu, v, delta);
  return v;
}

// ---------------------------------------------------------------------------------------------
// 16-byte (or scalar) vectors of T and conversion to / from fp32 lanes
// ---------------------------------------------------------------------------------------------
template <typename T, int VE>
struct alignas(sizeof(T) * VE) Pack {
  T v[VE];
};

template <typename T, int VE>
__device__ __forceinline__ void unpack(const Pack<T, VE>& p, float (&f)[VE]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int e = 0; e < VE; ++e) f[e] = p.v[e];
  } else if constexpr (VE % 2 == 0) {
#pragma unroll
    for (int e = 0; e < VE; e += 2) {
      if constexpr (std::is_same<T, __half>::value) {
        const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&p.v[e]));
        f[e] = t.x;
        f[e + 1] = t.y;
      } else {  // bf16 is the upper half of an fp32: one shift / one mask per pair
        const uint32_t w = *reinterpret_cast<const uint32_t*>(&p.v[e]);
        f[e] = __uint_as_float(w << 16);
        f[e + 1] = __uint_as_float(w & 0xffff0000u);
      }
    }
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      if constexpr (std::is_same<T, __half>::value)
        f[e] = __half2float(p.v[e]);
      else
        f[e] = __bfloat162float(p.v[e]);
    }
  }
}

template <typename T, int VE>
__device__ __forceinline__ Pack<T, VE> pack(const float (&f)[VE]) {
  Pack<T, VE> p;
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int e = 0; e < VE; ++e) p.v[e] = f[e];
  } else if constexpr (VE % 2 == 0) {
#pragma unroll
    for (int e = 0; e < VE; e += 2) {
      if constexpr (std::is_same<T, __half>::value)
        *reinterpret_cast<__half2*>(&p.v[e]) = __floats2half2_rn(f[e], f[e + 1]);
      else
        *reinterpret_cast<__nv_bfloat162*>(&p.v[e]) = __floats2bfloat162_rn(f[e], f[e + 1]);
    }
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      if constexpr (std::is_same<T, __half>::value)
        p.v[e] = __float2half_rn(f[e]);
      else
        p.v[e] = __float2bfloat16_rn(f[e]);
    }
  }
  return p;
}

template <typename T>
__device__ __forceinline__ float load_param(const T* p, int i) {
  if constexpr (sizeof(T) == 4)
    return p[i];
  else if constexpr (std::is_same<T, __half>::value)
    return __half2float(p[i]);
  else
    return __bfloat162float(p[i]);
}

// VE consecutive parameters starting at channel c (c is a multiple of VE on the vector path)
template <typename T, int VE>
__device__ __forceinline__ void load_params(const T* p, int c, float (&f)[VE]) {
  if constexpr (sizeof(T) * VE == 16) {
    Pack<T, VE> v;
    *reinterpret_cast<uint4*>(&v) = *reinterpret_cast<const uint4*>(p + c);
    unpack<T, VE>(v, f);
  } else {
#pragma unroll
    for (int e = 0; e < VE; ++e) f[e] = load_param<T>(p, c + e);
  }
}

template <typename T>
__device__ __forceinline__ T store_param(float v) {
  if constexpr (sizeof(T) == 4)
    return v;
  else if constexpr (std::is_same<T, __half>::value)
    return __float2half_rn(v);
  else
    return __float2bfloat16_rn(v);
}

// Global loads / stores with cache hints.  Streaming data is read once per pass; results are
// written once and not read again by this library.
template <typename V>
__device__ __forceinline__ V ld_stream(const V* p) {
  if constexpr (sizeof(V) == 16) {
    V out;
    *reinterpret_cast<uint4*>(&out) = *reinterpret_cast<const uint4*>(p);
    return out;
  } else {
    return *p;
  }
}
template <typename V>
__device__ __forceinline__ void st_stream(V* p, const V& v) {
  if constexpr (sizeof(V) == 16)
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&v);
  else
    *p = v;
}

// Shared memory by 32-bit shared-window address: explicit 128-bit accesses, asynchronous
// 16-byte global -> shared copies (no registers held while in flight).
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, const uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_dst), "l"(gmem_src) : "memory");
}
// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization
// attribute may become resident while its predecessor in the stream is still running: everything
// it does before grid_dep_wait() overlaps the predecessor's tail, and grid_dep_wait() returns once
// the predecessor grid has completed and its writes are visible.  grid_dep_launch_dependents() in
// the predecessor says "my CTA no longer minds sharing the SM"; CTAs that never call it count as
// having called it when they exit.  Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// wait until at most `pending` of the most recent commit groups are still in flight (pending <= 3)
__device__ __forceinline__ void cp_async_wait_dyn(int pending) {
  if (pending >= 3)
    cp_async_wait<3>();
  else if (pending == 2)
    cp_async_wait<2>();
  else if (pending == 1)
    cp_async_wait<1>();
  else
    cp_async_wait<0>();
}

// the same for pending <= 8
__device__ __forceinline__ void cp_async_wait_dyn8(int pending) {
  switch (pending) {
    case 0: cp_async_wait<0>(); break;
    case 1: cp_async_wait<1>(); break;
    case 2: cp_async_wait<2>(); break;
    case 3: cp_async_wait<3>(); break;
    case 4: cp_async_wait<4>(); break;
    case 5: cp_async_wait<5>(); break;
    case 6: cp_async_wait<6>(); break;
    case 7: cp_async_wait<7>(); break;
    default: cp_async_wait<8>(); break;
  }
}

// ---------------------------------------------------------------------------------------------
// Mixed-precision arithmetic of sm_100: one instruction converts a 16-bit operand and combines it
// with fp32 operands (PTX add / sub / fma with types .f32.f16 and .f32.bf16), so a 16-bit tensor
// element enters an fp32 sum without a separate unpack instruction.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void split_halves(uint32_t w, uint16_t& lo, uint16_t& hi) {
  asm("mov.b32 {%0, %1}, %2;" : "=h"(lo), "=h"(hi) : "r"(w));
}
// float(a) - c, exact conversion of a, one rounding
template <typename T>
__device__ __forceinline__ float mixed_sub(uint16_t a, float c) {
  static_assert(sizeof(T) == 2, "16-bit element types only");
  float d;
  if constexpr (std::is_same<T, __half>::value)
    asm("sub.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"(a), "f"(c));
  else
    asm("sub.rn.f32.bf16 %0, %1, %2;" : "=f"(d) : "h"(a), "f"(c));
  return d;
}
// float(a) + c
template <typename T>
__device__ __forceinline__ float mixed_add(uint16_t a, float c) {
  static_assert(sizeof(T) == 2, "16-bit element types only");
  float d;
  if constexpr (std::is_same<T, __half>::value)
    asm("add.rn.f32.f16 %0, %1, %2;" : "=f"(d) : "h"(a), "f"(c));
  else
    asm("add.rn.f32.bf16 %0, %1, %2;" : "=f"(d) : "h"(a), "f"(c));
  return d;
}
// float(a) * float(b) + c, product exact
template <typename T>
__device__ __forceinline__ float mixed_fma(uint16_t a, uint16_t b, float c) {
  static_assert(sizeof(T) == 2, "16-bit element types only");
  float d;
  if constexpr (std::is_same<T, __half>::value)
    asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
  else
    asm("fma.rn.f32.bf16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(b), "f"(c));
  return d;
}

// 16 bytes of T viewed as a uint4 <-> fp32 lanes
template <typename T, int VE>
__device__ __forceinline__ void unpack16(const uint4& w, float (&f)[VE]) {
  static_assert(sizeof(T) * VE == 16, "16-byte vectors only");
  const uint32_t r[4] = {w.x, w.y, w.z, w.w};
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int e = 0; e < 4; ++e) f[e] = __uint_as_float(r[e]);
  } else if constexpr (std::is_same<T, __half>::value) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&r[e]));
      f[2 * e] = t.x;
      f[2 * e + 1] = t.y;
    }
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      f[2 * e] = __uint_as_float(r[e] << 16);
      f[2 * e + 1] = __uint_as_float(r[e] & 0xffff0000u);
    }
  }
}
template <typename T, int VE>
__device__ __forceinline__ uint4 pack16(const float (&f)[VE]) {
  static_assert(sizeof(T) * VE == 16, "16-byte vectors only");
  uint32_t r[4];
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int e = 0; e < 4; ++e) r[e] = __float_as_uint(f[e]);
  } else if constexpr (std::is_same<T, __half>::value) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __half2 h = __floats2half2_rn(f[2 * e], f[2 * e + 1]);
      r[e] = *reinterpret_cast<const uint32_t*>(&h);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
      r[e] = *reinterpret_cast<const uint32_t*>(&h);
    }
  }
  return make_uint4(r[0], r[1], r[2], r[3]);
}
__device__ __forceinline__ uint4 ldg128(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void stg128(void* p, const uint4 v) { *reinterpret_cast<uint4*>(p) = v; }

// ---------------------------------------------------------------------------------------------
// Activations and their derivatives, evaluated in fp32.
//   FAST = false (fp32 tensors): libdevice expf / tanhf / erff, IEEE division -> meets 1e-5.
//   FAST = true  (16-bit tensors): hardware approximations (tanh.approx, ex2.approx, rcp.approx)
//                whose error (<= ~5e-4) sits below the rounding of a 16-bit result.
// Formulas: relu / silu / gelu(erf) / gelu(tanh) and derivatives as in gn_kernel.cu:62-106 of the
// reference.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float tanh_fast(float v) {
  float r;
  asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float ex2_fast(float v) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float rcp_fast(float v) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}

// Fast path of the erf-GELU: the normal CDF written as Phi(v) = 0.5 (1 + tanh(u(v))) with
// u(v) = v (c1 + c3 v^2 + c5 v^4), coefficients from a least-squares fit of Phi and of its
// derivative on [-8, 8] (max error 2.6e-5 in Phi, 1.1e-4 in Phi'); v^2 is clamped to 64 inside the
// polynomial, beyond which tanh has saturated.  One MUFU op (tanh.approx) per value.
constexpr float kPhiC1 = 7.97667873e-01f, kPhiC3 = 3.68576979e-02f, kPhiC5 = -3.17788673e-04f;

template <int ACT, bool FAST>
__device__ __forceinline__ float act_fwd(float v) {
  if constexpr (ACT == kActIdentity) {
    return v;
  } else if constexpr (ACT == kActRelu) {
    return v > 0.f ? v : 0.f;
  } else if constexpr (ACT == kActSilu) {
    if constexpr (FAST) {
      const float h = 0.5f * v;  // v * sigmoid(v) = h * tanh(h) + h
      return fmaf(h, tanh_fast(h), h);
    } else {
      return v / (1.0f + expf(-v));
    }
  } else if constexpr (ACT == kActGelu) {
    if constexpr (FAST) {
      const float v2 = fminf(v * v, 64.0f);
      const float t = tanh_fast(v * fmaf(fmaf(kPhiC5, v2, kPhiC3), v2, kPhiC1));
      const float h = 0.5f * v;
      return fmaf(h, t, h);
    } else {
      return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
    }
  } else {
    const float kBeta = 0.79788456080286536f;  // sqrt(2/pi)
    const float inner = kBeta * fmaf(0.044715f * v * v, v, v);
    const float h = 0.5f * v;
    if constexpr (FAST)
      return fmaf(h, tanh_fast(inner), h);
    else
      return fmaf(h, tanhf(inner), h);
  }
}

// d act(v) / dv
template <int ACT, bool FAST>
__device__ __forceinline__ float act_grad(float v) {
  if constexpr (ACT == kActIdentity) {
    return 1.0f;
  } else if constexpr (ACT == kActRelu) {
    return v > 0.f ? 1.0f : 0.f;
  } else if constexpr (ACT == kActSilu) {
    float s;
    if constexpr (FAST)
      s = fmaf(0.5f, tanh_fast(0.5f * v), 0.5f);
    else
      s = 1.0f / (1.0f + expf(-v));
    return s * fmaf(v, 1.0f - s, 1.0f);
  } else if constexpr (ACT == kActGelu) {
    if constexpr (FAST) {
      const float v2 = fminf(v * v, 64.0f);
      const float t = tanh_fast(v * fmaf(fmaf(kPhiC5, v2, kPhiC3), v2, kPhiC1));
      const float du = fmaf(fmaf(5.0f * kPhiC5, v2, 3.0f * kPhiC3), v2, kPhiC1);
      // Phi + v * Phi',  Phi' = 0.5 (1 - t^2) u'; beyond |v| = 8 tanh saturates and the second term is 0
      return fmaf(0.5f * v * du, fmaf(-t, t, 1.0f), fmaf(0.5f, t, 0.5f));
    } else {
      const float kInvSqrt2Pi = 0.39894228040143268f;
      const float cdf = 0.5f * (1.0f + erff(v * 0.70710678118654752f));
      const float pdf = expf(-0.5f * v * v) * kInvSqrt2Pi;
      return fmaf(v, pdf, cdf);
    }
  } else {
    const float kBeta = 0.79788456080286536f;
    const float v2 = v * v;
    const float inner = kBeta * fmaf(0.044715f * v2, v, v);
    float t;
    if constexpr (FAST)
      t = tanh_fast(inner);
    else
      t = tanhf(inner);
    const float dinner = kBeta * fmaf(3.0f * 0.044715f, v2, 1.0f);
    // 0.5 (1 + t) + 0.5 v (1 - t^2) dinner
    return fmaf(0.5f * v * dinner, fmaf(-t, t, 1.0f), fmaf(0.5f, t, 0.5f));
  }
}

// ---------------------------------------------------------------------------------------------
// Packed f16x2 evaluation of the smooth activations for 16-bit tensors: two channels per
// instruction and per MUFU op.  The pre-activation yh is formed in fp32 and converted with
// saturation (|yh| > 65504 clamps instead of becoming inf); what is evaluated in half precision
// (11 significant bits) is only the activation, whose result is rounded to a 16-bit tensor anyway
// (forward) or multiplies a 16-bit dy (backward).  fp32 tensors never take this path.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ __half2 f32x2_to_h2_sat(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return *reinterpret_cast<__half2*>(&r);
}
__device__ __forceinline__ __half2 tanh_h2(__half2 v) {
  uint32_t r;
  asm("tanh.approx.f16x2 %0, %1;" : "=r"(r) : "r"(*reinterpret_cast<uint32_t*>(&v)));
  return *reinterpret_cast<__half2*>(&r);
}

// which (activation, tensor type) pairs use the packed path: where it saves instructions
template <typename T, int ACT>
__host__ __device__ constexpr bool use_h2_fwd() {
  return sizeof(T) == 2 && (ACT == kActGelu || ACT == kActGeluTanh || (ACT == kActSilu && std::is_same<T, __half>::value));
}
template <typename T, int ACT>
__host__ __device__ constexpr bool use_h2_bwd() {
  return sizeof(T) == 2 && (ACT == kActGelu || ACT == kActGeluTanh || ACT == kActSilu);
}

// tanh argument u(v) and its derivative du/dv for the two GELU forms, v^2 clamped to 64
template <int ACT>
__device__ __forceinline__ void gelu_poly_h2(__half2 v, __half2& u, __half2& du, bool want_du) {
  const __half2 v2 = __hmin2(__hmul2(v, v), __float2half2_rn(64.0f));
  if constexpr (ACT == kActGelu) {
    const __half2 c1 = __float2half2_rn(kPhiC1), c3 = __float2half2_rn(kPhiC3), c5 = __float2half2_rn(kPhiC5);
    u = __hmul2(v, __hfma2(__hfma2(c5, v2, c3), v2, c1));
    if (want_du)
      du = __hfma2(__hfma2(__float2half2_rn(5.0f * kPhiC5), v2, __float2half2_rn(3.0f * kPhiC3)), v2, c1);
  } else {
    const float kBeta = 0.79788456080286536f;
    u = __hmul2(v, __hfma2(__float2half2_rn(kBeta * 0.044715f), v2, __float2half2_rn(kBeta)));
    if (want_du) du = __hfma2(__float2half2_rn(3.0f * kBeta * 0.044715f), v2, __float2half2_rn(kBeta));
  }
}

template <int ACT>
__device__ __forceinline__ __half2 act_fwd_h2(__half2 v) {
  const __half2 half_ = __float2half2_rn(0.5f);
  if constexpr (ACT == kActSilu) {
    const __half2 h = __hmul2(v, half_);
    return __hfma2(h, tanh_h2(h), h);
  } else {
    __half2 u, du;
    gelu_poly_h2<ACT>(v, u, du, false);
    const __half2 h = __hmul2(v, half_);
    return __hfma2(h, tanh_h2(u), h);
  }
}

template <int ACT>
__device__ __forceinline__ __half2 act_grad_h2(__half2 v) {
  const __half2 half_ = __float2half2_rn(0.5f), one = __float2half2_rn(1.0f);
  if constexpr (ACT == kActRelu) {
    return __hgt2(v, __float2half2_rn(0.0f));  // 1.0 where v > 0, else 0.0
  } else if constexpr (ACT == kActSilu) {
    const __half2 t = tanh_h2(__hmul2(v, half_));
    const __half2 s = __hfma2(half_, t, half_);
    return __hmul2(s, __hfma2(v, __hsub2(one, s), one));
  } else {
    __half2 u, du;
    gelu_poly_h2<ACT>(v, u, du, true);
    const __half2 t = tanh_h2(u);
    // Phi + v * Phi' with Phi' = 0.5 (1 - t^2) u'.  The factor (1 - t^2) is applied before u': for
    // |v| beyond a few tens it is exactly 0, so the product cannot overflow to inf (and inf * 0 = NaN)
    // when v * u' exceeds the half-precision range (|v| above about 1.7e4).
    return __hfma2(__hmul2(__hmul2(v, half_), __hfma2(__hneg2(t), t, one)), du, __hfma2(half_, t, half_));
  }
}

// Forward epilogue for one 16-byte vector: out = T(act(yh)) packed.
template <typename T, int VE, int ACT>
__device__ __forceinline__ uint4 act_pack16(const float (&yh)[VE]) {
  if constexpr (use_h2_fwd<T, ACT>()) {
    uint32_t r[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __half2 y = act_fwd_h2<ACT>(f32x2_to_h2_sat(yh[2 * e], yh[2 * e + 1]));
      if constexpr (std::is_same<T, __half>::value) {
        r[e] = *reinterpret_cast<const uint32_t*>(&y);
      } else {
        const float2 f = __half22float2(y);
        const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
        r[e] = *reinterpret_cast<const uint32_t*>(&b);
      }
    }
    return make_uint4(r[0], r[1], r[2], r[3]);
  } else {
    constexpr bool FAST = sizeof(T) == 2;
    float o[VE];
#pragma unroll
    for (int e = 0; e < VE; ++e) o[e] = act_fwd<ACT, FAST>(yh[e]);
    return pack16<T, VE>(o);
  }
}

// Backward: g[e] = act'(yh[e]) for one vector.
template <typename T, int VE, int ACT>
__device__ __forceinline__ void act_grad_vec(const float (&yh)[VE], float (&g)[VE]) {
  if constexpr (use_h2_bwd<T, ACT>() && VE % 2 == 0) {
#pragma unroll
    for (int e = 0; e < VE; e += 2) {
      const float2 f = __half22float2(act_grad_h2<ACT>(f32x2_to_h2_sat(yh[e], yh[e + 1])));
      g[e] = f.x;
      g[e + 1] = f.y;
    }
  } else {
    constexpr bool FAST = sizeof(T) == 2;
#pragma unroll
    for (int e = 0; e < VE; ++e) g[e] = act_grad<ACT, FAST>(yh[e]);
  }
}

// ---------------------------------------------------------------------------------------------
// Thread-block cluster helpers (raw PTX so arrive and wait can be split)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned cluster_ctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ unsigned cluster_nctarank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
// Arrival without memory ordering of its own (pairs with a preceding fence where one is needed);
// unlike the release form it does not wait for the CTA's outstanding stores.
__device__ __forceinline__ void cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// ---------------------------------------------------------------------------------------------
// Exchange between the CTAs of a cluster without a cluster barrier: every CTA pushes its values
// into its peers' shared memory with st.async, which also counts the bytes on an mbarrier of the
// receiving CTA; the receiver waits for the byte count.  No fence is involved, so the exchange
// does not wait for the CTA's outstanding global stores as a release barrier would.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void fence_mbar_init_cluster() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// one arrival of this thread plus the announcement that `bytes` will be delivered by st.async
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Where a wait that gave up is recorded: a device counter (read by gnb200_wait_timeouts) and a
// word of mapped pinned host memory that the entry points look at, without synchronising, before
// they launch anything.
struct WaitLimit {
  unsigned int* timeouts;      // device counter of waits that gave up
  unsigned int* host_mirror;   // mapped host word, set non-zero together with the counter
  long long clocks;            // give up after this many SM clocks ...
  unsigned int polls;          // ... and at least this many failed polls (a context that was switched
                               // out lets the clock run on, but polls only count while it executes)
};
__device__ __forceinline__ void wait_gave_up(const WaitLimit& lim) {
  atomicAdd(lim.timeouts, 1u);
  *reinterpret_cast<volatile unsigned int*>(lim.host_mirror) = 1u;
  __threadfence_system();
}
// Waits for the phase with the given parity.  Returns false if the wait gave up (both limits of
// `lim` exceeded); the give-up is recorded and the caller must treat what it waited for as missing.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, unsigned parity, const WaitLimit& lim) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  unsigned int polls = 0;
  while (!mbar_try_wait(bar, parity)) {
    ++polls;
    if (polls > lim.polls && clock64() - t0 > lim.clocks) {
      wait_gave_up(lim);
      return false;
    }
  }
  return true;
}
// announces `bytes` more st.async bytes on the current phase without arriving
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// 16 bytes into the shared memory of CTA `rank` at the offset of `local_dst`, counted on that
// CTA's mbarrier at the offset of `local_bar`
__device__ __forceinline__ void st_async_f32x4(float* local_dst, uint64_t* local_bar, unsigned rank, float a, float b,
                                               float c, float d) {
  uint32_t rdst, rbar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rdst) : "r"(smem_addr(local_dst)), "r"(rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rbar) : "r"(smem_addr(local_bar)), "r"(rank));
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(rdst),
               "r"(__float_as_uint(a)), "r"(__float_as_uint(b)), "r"(__float_as_uint(c)), "r"(__float_as_uint(d)),
               "r"(rbar)
               : "memory");
}

// ---------------------------------------------------------------------------------------------
// Geometry of one launch, filled in by the host planner
// ---------------------------------------------------------------------------------------------
// Division by a launch-time constant d (1 <= d < 2^31) for 0 <= n < 2^31:
// n / d == (umulhi(n, mul) + n) >> shr.  Filled in by the host planner.
struct FastDiv {
  uint32_t mul, shr;
  __device__ __forceinline__ int div(int n) const { return (int)((__umulhi((uint32_t)n, mul) + (uint32_t)n) >> shr); }
};

struct Geom {
  int N, R, C, G, D;
  int CW;            // channels per column block (multiple of VE)
  int CV;            // CW / VE: vectors per tile row == threads along C
  int TY;            // row lanes; CV * TY threads do the streaming work
  int ncb;           // column blocks per sample
  int rows_per_cta;  // pixels per CTA tile
  int chunks;        // CTA tiles per (sample, column block): ceil(R / rows_per_cta)
  int slots;         // upper bound on the groups a column block touches
  int k;             // cluster size of the fused kernels (== chunks there)
  FastDiv div_D, div_CV, div_CW, div_ncb, div_chunks;
  // Shuffle reductions (fused kernels): usable when every vector lies in one group, CV and the
  // threads per group row (D / VE) are powers of two and CV <= 32.  tps_shift = log2(D / VE).
  int shuf, tps_shift;
  int red_floats;  // size of the reduction scratch `red`, set by the planner
  int wsum_stride, wpart_off;  // shuffle reductions: second warp-sum buffer and (backward) per-warp channel sums in `red`, in floats
  WaitLimit wait;  // limits and give-up record of the bounded waits (set by the launcher)
  int skip_push_rank;  // -1; the exchange self-test names a cluster rank that withholds its pushes
  int persist;     // fused forward: the grid holds the resident clusters only, each looping over items
};

// Geometry of the wave plan (gn_wave.cu): a persistent cooperative kernel that takes the tensor
// through both passes wave by wave.  A wave is a range of `ipw` (sample, column block) slabs
// ("items"); every item is cut into `chunks` row chunks ("units") that are dealt to the CTAs.
constexpr int kWaveConsumers = 256;                 // consumer threads of a wave CTA
constexpr int kWaveThreads = kWaveConsumers + 32;   // plus the producer warp
struct WaveGeom {
  int N, R, C, G, D;
  int CW, CV, TY;      // channels / 16-byte vectors per column block row; row lanes of the consumers
  int ncb, slots;      // column blocks per sample; groups per column block
  int KR, BR;          // rows per consumer thread and rows per TMA box of one stage (BR = KR * TY)
  int stages;          // depth of the shared-memory ring
  int box_bytes;       // BR * CW * sizeof(T)
  int stage_bytes;     // box_bytes rounded up to 128 (TMA destinations are 128-byte aligned)
  int chunks, rows_per_chunk;  // units per item; rows per unit (a multiple of BR)
  int items, ipw, waves;
  int consumers;       // consumer threads (a multiple of 32)
  int overlap;         // pass A of the next wave runs before pass B of this one (two waves share L2)
  int teams;           // the CTAs form this many teams that take alternate waves independently
  FastDiv div_D, div_CV, div_ncb;
  WaitLimit wait;
  unsigned long long* trace;  // optional timeline buffer (tuning aid), else null
};

// Groups touched by column block starting at channel c0 (width CW, clipped to C):
// first group and how many.
__device__ __forceinline__ void cb_groups(const Geom& g, int c0, int& g_lo, int& n_slots) {
  const int c_end = min(c0 + g.CW, g.C);
  g_lo = g.div_D.div(c0);
  n_slots = g.div_D.div(c_end - 1) - g_lo + 1;
}

// ---------------------------------------------------------------------------------------------
// CTA-level reductions.  Every order of summation is fixed by the launch geometry (no atomics),
// so results are bit-identical from run to run.
// ---------------------------------------------------------------------------------------------

// Sum of NV values per streaming thread over the CTA tile, per group slot of the column block.
//   NV == VE : one value per channel (a vector may straddle groups)
//   NV == 1  : one value per thread (every vector lies inside one group: D % VE == 0)
//   val[i]   : must be 0 for threads that did not stream
//   red      : TY * CV * NV floats of shared scratch;  out[s], s < n_slots : shared, valid on return
template <int VE, int NV>
__device__ __forceinline__ void cta_group_sum(const Geom& g, const float (&val)[NV], int tx, int ty, int c0, int g_lo,
                                              int n_slots, float* red, float* out) {
  const int TY = g.TY;
  const int cols = g.CV * NV;  // values per row lane
  if (ty < TY) {
#pragma unroll
    for (int e = 0; e < NV; ++e) red[ty * cols + tx * NV + e] = val[e];
  }
  __syncthreads();
  const int c_valid = min(g.CW, g.C - c0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = (blockDim.x + 31) >> 5;
  for (int s = warp; s < n_slots; s += nwarps) {
    int lo = max((g_lo + s) * g.D, c0) - c0;
    int hi = min((g_lo + s + 1) * g.D, c0 + c_valid) - c0;
    if (NV == 1) {  // channels -> vectors (group boundaries are multiples of VE here)
      lo /= VE;
      hi /= VE;
    }
    const int w = hi - lo;
    // lanes form a (32 / w2) x w2 grid over (row lane, column), w2 = power of two >= min(w, 32)
    int sh = 0;
    while ((1 << sh) < w && sh < 5) ++sh;
    const int cl = lane & ((1 << sh) - 1), jl = lane >> sh, jstep = 32 >> sh;
    float acc = 0.f;
    for (int j = jl; j < TY; j += jstep)
      for (int c = cl; c < w; c += (1 << sh)) acc += red[j * cols + lo + c];
    acc = warp_sum(acc);
    if (lane == 0) out[s] = acc;
  }
  __syncthreads();
}

// Sum of one value per thread over the CTA, per group slot, for the shuffle geometry (Geom::shuf):
// lanes of a warp that share a slot are combined with xor-butterflies (identical result in every
// lane), warp results go through `wsum` (nwarps * n_slots floats) and are added in warp order.
// Returns the total of the calling thread's own slot; one __syncthreads inside.  Two consecutive
// calls must use different `wsum` buffers.
__device__ __forceinline__ float cta_slot_sum_shuf(const Geom& g, float v, int tx, float* wsum) {
  const int tps = 1 << g.tps_shift;
  for (int b = 1; b < tps; b <<= 1) v += __shfl_xor_sync(0xffffffffu, v, b);
  for (int b = g.CV; b < 32; b <<= 1) v += __shfl_xor_sync(0xffffffffu, v, b);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  const int n_slots = g.CV >> g.tps_shift;
  if (lane < g.CV && (lane & (tps - 1)) == 0) wsum[warp * n_slots + (lane >> g.tps_shift)] = v;
  __syncthreads();
  const int s = tx >> g.tps_shift;
  float t = 0.f;
  for (int w = 0; w < nwarps; ++w) t += wsum[w * n_slots + s];
  return t;
}

// Per-channel sums over the row lanes of two values (backward): chan[c] = sum_ty s1, chan[CW + c]
// = sum_ty s2.  red: 2 * TY * CW floats, part: 2 * J * CW floats with J = max(1, blockDim / CW).
template <int VE>
__device__ __forceinline__ void cta_channel_sums(const Geom& g, const float (&s1)[VE], const float (&s2)[VE], int tx,
                                                 int ty, int c0, float* red, float* part, float* chan) {
  const int CW = g.CW, TY = g.TY;
  float* red1 = red;
  float* red2 = red + TY * CW;
  if (ty < TY) {
    if constexpr (VE % 4 == 0) {  // 16-byte stores: no bank conflicts (CW is a multiple of VE)
#pragma unroll
      for (int e = 0; e < VE; e += 4) {
        *reinterpret_cast<float4*>(red1 + ty * CW + tx * VE + e) = make_float4(s1[e], s1[e + 1], s1[e + 2], s1[e + 3]);
        *reinterpret_cast<float4*>(red2 + ty * CW + tx * VE + e) = make_float4(s2[e], s2[e + 1], s2[e + 2], s2[e + 3]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        red1[ty * CW + tx * VE + e] = s1[e];
        red2[ty * CW + tx * VE + e] = s2[e];
      }
    }
  }
  __syncthreads();
  const int J = max(1, (int)blockDim.x / CW);  // row-lane slices summed in parallel
  {
    const int j = (int)blockDim.x >= CW ? g.div_CW.div((int)threadIdx.x) : 0;
    if (j < J) {
      for (int c = threadIdx.x - j * CW; c < CW; c += blockDim.x) {  // one pass unless CW > blockDim
        float a1 = 0.f, a2 = 0.f;
        for (int r = j; r < TY; r += J) {
          a1 += red1[r * CW + c];
          a2 += red2[r * CW + c];
        }
        part[j * CW + c] = a1;
        part[(J + j) * CW + c] = a2;
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < CW; c += blockDim.x) {
    float a1 = 0.f, a2 = 0.f;
    for (int j = 0; j < J; ++j) {
      a1 += part[j * CW + c];
      a2 += part[(J + j) * CW + c];
    }
    chan[c] = a1;
    chan[CW + c] = a2;
  }
  __syncthreads();
}

// The same for the shuffle geometry (Geom::shuf), without the TY x CW staging area: lanes of a warp
// that hold the same column vector (equal lane mod CV) are combined with xor-butterflies, the warp
// sums go through `wpart` (nwarps * 2 * CW floats) and thread c < c_valid adds them in warp order
// and stores (S1, S2) of channel c to out[c].  One __syncthreads inside.
template <int VE>
__device__ __forceinline__ void cta_channel_sums_shuf(const Geom& g, const float (&s1)[VE], const float (&s2)[VE],
                                                      int tx, float* wpart, float2* out, int c_valid) {
  static_assert(VE % 4 == 0, "vector path only");
  float v1[VE], v2[VE];
#pragma unroll
  for (int e = 0; e < VE; ++e) v1[e] = s1[e], v2[e] = s2[e];
  for (int b = g.CV; b < 32; b <<= 1) {
#pragma unroll
    for (int e = 0; e < VE; ++e) {
      v1[e] += __shfl_xor_sync(0xffffffffu, v1[e], b);
      v2[e] += __shfl_xor_sync(0xffffffffu, v2[e], b);
    }
  }
  const int CW = g.CW;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  if (lane < g.CV) {
    float* w1 = wpart + (size_t)(2 * warp) * CW + tx * VE;
    float* w2 = w1 + CW;
#pragma unroll
    for (int e = 0; e < VE; e += 4) {
      *reinterpret_cast<float4*>(w1 + e) = make_float4(v1[e], v1[e + 1], v1[e + 2], v1[e + 3]);
      *reinterpret_cast<float4*>(w2 + e) = make_float4(v2[e], v2[e + 1], v2[e + 2], v2[e + 3]);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < c_valid; c += blockDim.x) {
    float a1 = 0.f, a2 = 0.f;
    for (int w = 0; w < nwarps; ++w) {
      a1 += wpart[(size_t)(2 * w) * CW + c];
      a2 += wpart[(size_t)(2 * w + 1) * CW + c];
    }
    out[c] = make_float2(a1, a2);
  }
}

}  // namespace gnb200
