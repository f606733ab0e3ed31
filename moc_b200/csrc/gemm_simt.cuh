// CUDA-core GEMM with fp32 accumulation and arbitrary operand strides, used for fp32
// tensors (the tensor-core core is bf16 only) and as an independent cross-check of the
// tcgen05 core in the tests. Same contract as the tcgen05 core: C[M,N] = sum over up to
// two K segments of A_s[M,K_s] * B_s[N,K_s]^T, same epilogue functors (one thread = one
// row x 32 columns).
#pragma once

#include "common.cuh"
#include "epilogues.cuh"

namespace moc {

template <typename T>
struct SimtOperand {
  const T* p;
  int64_t s_mn;   // element stride along M (for A) or N (for B)
  int64_t s_k;    // element stride along K
};

constexpr int kSimtBM = 64;
constexpr int kSimtBN = 64;
constexpr int kSimtBK = 16;
constexpr int kSimtThreads = 128;

template <typename T>
__device__ __forceinline__ void simt_load_tile(const SimtOperand<T>& op, int mn0, int mn_max, int k0, int k_max,
                                               float (*dst)[kSimtBM + 4]) {
  // 64 (mn) x 16 (k) elements, 8 per thread; walk the contiguous dimension fastest
  const int t = threadIdx.x;
  if (op.s_k == 1) {
    const int kk = t & 15;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = (t >> 4) + 8 * i;
      const int mn = mn0 + r, k = k0 + kk;
      float v = 0.0f;
      if (mn < mn_max && k < k_max) v = Num<T>::to_float(op.p[mn * op.s_mn + k]);
      dst[kk][r] = v;
    }
  } else {
    const int r = t & 63;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int kk = (t >> 6) + 2 * i;
      const int mn = mn0 + r, k = k0 + kk;
      float v = 0.0f;
      if (mn < mn_max && k < k_max) v = Num<T>::to_float(op.p[mn * op.s_mn + k * op.s_k]);
      dst[kk][r] = v;
    }
  }
}

template <typename T, class Epi>
__global__ void __launch_bounds__(kSimtThreads)
gemm_simt_kernel(SimtOperand<T> a0, SimtOperand<T> b0, int k0_len, SimtOperand<T> a1, SimtOperand<T> b1, int k1_len,
                 int m, int n, int group, const Epi epi) {
  __shared__ __align__(16) float as[kSimtBK][kSimtBM + 4];
  __shared__ __align__(16) float bs[kSimtBK][kSimtBN + 4];
  const int m0 = blockIdx.y * kSimtBM;
  const int n0 = blockIdx.x * kSimtBN;
  const int r = threadIdx.x >> 1;          // row within the tile
  const int h = (threadIdx.x & 1) * 32;    // column half
  float acc[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) acc[j] = 0.0f;

  for (int seg = 0; seg < 2; ++seg) {
    const SimtOperand<T>& a = seg ? a1 : a0;
    const SimtOperand<T>& b = seg ? b1 : b0;
    const int klen = seg ? k1_len : k0_len;
    for (int k0 = 0; k0 < klen; k0 += kSimtBK) {
      simt_load_tile<T>(a, m0, m, k0, klen, as);
      simt_load_tile<T>(b, n0, n, k0, klen, bs);
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < kSimtBK; ++kk) {
        const float av = as[kk][r];
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) {
          const float4 bv = *reinterpret_cast<const float4*>(&bs[kk][h + 4 * j4]);
          acc[4 * j4 + 0] = fmaf(av, bv.x, acc[4 * j4 + 0]);
          acc[4 * j4 + 1] = fmaf(av, bv.y, acc[4 * j4 + 1]);
          acc[4 * j4 + 2] = fmaf(av, bv.z, acc[4 * j4 + 2]);
          acc[4 * j4 + 3] = fmaf(av, bv.w, acc[4 * j4 + 3]);
        }
      }
      __syncthreads();
    }
  }
  const int row = m0 + r, col0 = n0 + h;
  if (row < m && col0 < n) {
    typename Epi::Ctx ctx;
    epi.begin(ctx, group, row, col0, 1);
    epi.prefetch(ctx, row, col0, 0);
    epi(ctx, group, row, col0, 0, acc);
  }
}

}  // namespace moc
