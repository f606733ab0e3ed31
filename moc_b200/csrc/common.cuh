// Shared device/host helpers for the MoC sparse SwiGLU FFN kernels (sm_100a).
//
// Numeric conventions follow the reference training path (moc/ffn.py:124-259 and
// moc/training/triton_sparse_aux.py:17-49, :376-400): every intermediate that the
// reference materialises as a tensor is rounded to the storage type at the same
// point, so that bf16 results stay within one rounding step of the reference.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace moc {

// ---- status codes returned through the C ABI (negative = error) -------------
enum Status : int {
  kOk = 0,
  kErrInvalidArg = -1,      // null pointer, bad size, unsupported dtype
  kErrUnsupported = -2,     // shape outside what the kernels handle
  kErrWorkspace = -3,       // workspace too small or misaligned
  kErrCuda = -4,            // a CUDA runtime / driver call failed
  kErrTensorMap = -5,       // cuTensorMapEncodeTiled rejected a descriptor
  kErrDeviceTimeout = -6,   // a bounded device-side wait gave up (status word set)
};

// dtype codes of the C ABI
enum DType : int { kBF16 = 0, kF32 = 1 };

// Device status word layout: 0 = fine, otherwise (code << 24) | detail.
constexpr int kDevTimeoutProducer = 1;
constexpr int kDevTimeoutMma = 2;
constexpr int kDevTimeoutEpilogue = 3;

// ---- storage-type traits -------------------------------------------------------
template <typename T> struct Num;

template <> struct Num<__nv_bfloat16> {
  static constexpr bool kIsBf16 = true;
  __device__ __forceinline__ static float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ __forceinline__ static __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
  // value after a round trip through the storage type
  __device__ __forceinline__ static float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
  // storage value of a float that is already exactly representable (no conversion instruction)
  __device__ __forceinline__ static __nv_bfloat16 from_rounded(float v) {
    const uint16_t b = static_cast<uint16_t>(__float_as_uint(v) >> 16);
    return *reinterpret_cast<const __nv_bfloat16*>(&b);
  }
  // rounds two values with one packed conversion (the scalar conversion runs on the slow XU pipe)
  __device__ __forceinline__ static void round_pair(float& a, float& b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    const uint32_t w = *reinterpret_cast<const uint32_t*>(&h);
    a = __uint_as_float(w << 16);
    b = __uint_as_float(w & 0xFFFF0000u);
  }
};

template <> struct Num<float> {
  static constexpr bool kIsBf16 = false;
  __device__ __forceinline__ static float to_float(float v) { return v; }
  __device__ __forceinline__ static float from_float(float v) { return v; }
  __device__ __forceinline__ static float round(float v) { return v; }
  __device__ __forceinline__ static float from_rounded(float v) { return v; }
  __device__ __forceinline__ static void round_pair(float&, float&) {}
};

// Sigmoid evaluated in fp32 (SiLU(g) = g * sigmoid(g), moc/training/triton_sparse_aux.py:39).
// fp32 tensors: full-precision expf and IEEE division. bf16 tensors: ex2/rcp approximations
// (about 2 fp32 ulp), far below the bf16 rounding that follows; the same function is used
// wherever a value is recomputed, so forward and backward agree bit for bit.
template <typename T> __device__ __forceinline__ float sigmoid_act(float g);
template <> __device__ __forceinline__ float sigmoid_act<float>(float g) { return 1.0f / (1.0f + expf(-g)); }
template <> __device__ __forceinline__ float sigmoid_act<__nv_bfloat16>(float g) {
  return __fdividef(1.0f, 1.0f + __expf(-g));
}

// s = round(SiLU(g)) (moc/ffn.py:157)
template <typename T>
__device__ __forceinline__ float silu_round(float g) { return Num<T>::round(g * sigmoid_act<T>(g)); }

// Selected-channel forward math: s = round(SiLU(g)), z = round(s * u)
// (moc/training/triton_sparse_aux.py:39-45).
template <typename T>
__device__ __forceinline__ void moc_fwd_point(float g, float u, float& s, float& z) {
  s = silu_round<T>(g);
  z = Num<T>::round(s * u);
}

// Selected-channel backward math (moc/ffn.py:222-229 via
// moc/training/triton_sparse_aux.py:376-400): with storage type bf16 every step of
// SiLU' is rounded, as the chain of PyTorch bf16 ops does; in fp32 nothing is.
// s = round(SiLU(g)) is rebuilt from the same sigmoid evaluation.
template <typename T>
__device__ __forceinline__ void moc_bwd_point(float g, float u, float gz, float& grad_g, float& grad_u) {
  using N = Num<T>;
  const float sig_full = sigmoid_act<T>(g);
  const float s = N::round(g * sig_full);
  const float grad_s = N::round(u * gz);
  grad_u = N::round(s * gz);
  const float sig = N::round(sig_full);
  const float one_minus = N::round(1.0f - sig);
  const float g_term = N::round(g * one_minus);
  const float inner = N::round(1.0f + g_term);
  const float deriv = N::round(sig * inner);
  grad_g = N::round(grad_s * deriv);
}

// Order-preserving key maps: larger key <=> larger value under the IEEE total
// order (-0 < +0). Same map as bf16_order_key in
// moc/inference/cuda/optimized_global_moc_ext.cu:26-29, extended to fp32.
__device__ __host__ __forceinline__ uint32_t order_key16(uint16_t bits) {
  return (bits & 0x8000u) ? (uint32_t)(bits ^ 0xFFFFu) : (uint32_t)(bits ^ 0x8000u);
}
__device__ __host__ __forceinline__ uint32_t order_key32(uint32_t bits) {
  return (bits & 0x80000000u) ? ~bits : (bits ^ 0x80000000u);
}

__host__ __device__ __forceinline__ int64_t round_up_i64(int64_t v, int64_t m) { return (v + m - 1) / m * m; }
__host__ __device__ __forceinline__ int ceil_div_i(int a, int b) { return (a + b - 1) / b; }

// Leading dimension (elements) of the dense [tokens, d_ffn] scratch matrices: rows
// start on 128-byte boundaries and 32-column chunks never cross the row end.
__host__ __device__ __forceinline__ int64_t ffn_ld(int64_t d_ffn) { return round_up_i64(d_ffn, 128); }
// 32-bit words per row of the selection bitmap.
__host__ __device__ __forceinline__ int64_t mask_words(int64_t d_ffn) { return ffn_ld(d_ffn) / 32; }

}  // namespace moc
