// Matrix product on the CUDA cores with float accumulation: the true 32-bit path of every
// linear layer, and the fallback of the bfloat16 path for shapes the tensor-core kernel refuses.
//
//   out[m, n] = act(sum_k a[m, k] * w(k, n) + bias[n]) (+ residual[m, n])
//
// `w` is stored [K, N] (the Conv1D layout of GPT-2 checkpoints, x @ w:
// kelpie-models/kelpie_models/models/torch/gpt2.py:52-55) or [N, K] (a tied embedding used as
// the head, x @ wte^T: gpt2.py:101). Each output element is one thread's sum over k in
// ascending order, so a row's result does not depend on how many other rows the call has.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW, typename TO, bool W_IS_NK>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TA* __restrict__ a, int lda, const TW* __restrict__ w, int ldw,
                 const float* __restrict__ bias, const float* __restrict__ residual, int ldr,
                 TO* __restrict__ out, int ldo, int m_total, int n_total, int k_total, int act) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  __shared__ float as[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < k_total; k0 += BK) {
    // a tile: BM x BK, k fastest in memory
    for (int i = tid; i < BM * BK; i += 256) {
      int mm = i / BK, kk = i % BK;
      int gm = m0 + mm, gk = k0 + kk;
      as[kk][mm] = (gm < m_total && gk < k_total) ? to_float(a[size_t(gm) * lda + gk]) : 0.f;
    }
    if (W_IS_NK) {
      for (int i = tid; i < BN * BK; i += 256) {
        int nn = i / BK, kk = i % BK;
        int gn = n0 + nn, gk = k0 + kk;
        ws[kk][nn] = (gn < n_total && gk < k_total) ? to_float(w[size_t(gn) * ldw + gk]) : 0.f;
      }
    } else {
      for (int i = tid; i < BN * BK; i += 256) {
        int kk = i / BN, nn = i % BN;
        int gn = n0 + nn, gk = k0 + kk;
        ws[kk][nn] = (gn < n_total && gk < k_total) ? to_float(w[size_t(gk) * ldw + gn]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[TM], wv[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) av[i] = as[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) wv[j] = ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int gm = m0 + ty * TM + i;
    if (gm >= m_total) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      int gn = n0 + tx * TN + j;
      if (gn >= n_total) continue;
      float v = acc[i][j];
      if (bias != nullptr) v += bias[gn];
      v = activate(v, act);
      if (residual != nullptr) v += residual[size_t(gm) * ldr + gn];
      out[size_t(gm) * ldo + gn] = from_float<TO>(v);
    }
  }
}

template <typename TA, typename TW, typename TO>
int launch(const void* a, int lda, const void* w, int ldw, int w_is_nk, const float* bias, const float* residual,
           int ldr, void* out, int ldo, int m, int n, int k, int act, cudaStream_t stream) {
  dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
  if (w_is_nk) {
    r2_launch(gemm_simt_kernel<TA, TW, TO, true>, dim3(grid), dim3(256), size_t(0), stream, (const TA*)a, lda, (const TW*)w, ldw, bias, residual,
                                                                 ldr, (TO*)out, ldo, m, n, k, act);
  } else {
    r2_launch(gemm_simt_kernel<TA, TW, TO, false>, dim3(grid), dim3(256), size_t(0), stream, (const TA*)a, lda, (const TW*)w, ldw, bias, residual,
                                                                  ldr, (TO*)out, ldo, m, n, k, act);
  }
  return launch_status();
}

}  // namespace

// a [m, k] (leading dimension lda), w [k, n] or [n, k] (ldw), bias [n] float or null,
// residual [m, n] float or null (ldr), out [m, n] (ldo). Activations and weights share a dtype.
extern "C" int r2_gemm_simt(const void* a, int lda, const void* w, int ldw, int w_is_nk, const float* bias,
                            const float* residual, int ldr, void* out, int ldo, int m, int n, int k, int act,
                            int in_dtype, int out_dtype, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return R2_OK;
  if (k < 1) return R2_BAD_SHAPE;
  if (act < R2_ACT_NONE || act > R2_ACT_GELU_ERF) return R2_UNSUPPORTED;
  if (in_dtype == R2_F32 && out_dtype == R2_F32)
    return launch<float, float, float>(a, lda, w, ldw, w_is_nk, bias, residual, ldr, out, ldo, m, n, k, act, stream);
  if (in_dtype == R2_BF16 && out_dtype == R2_F32)
    return launch<bf16, bf16, float>(a, lda, w, ldw, w_is_nk, bias, residual, ldr, out, ldo, m, n, k, act, stream);
  if (in_dtype == R2_BF16 && out_dtype == R2_BF16)
    return launch<bf16, bf16, bf16>(a, lda, w, ldw, w_is_nk, bias, residual, ldr, out, ldo, m, n, k, act, stream);
  return R2_BAD_DTYPE;
}
