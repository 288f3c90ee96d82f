// Row-wise kernels: token embedding (+ learned positions), LayerNorm, and the write of new
// keys and values into their cache pages. All statistics and sums are in float.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// x[t] = table[ids[t]] (+ pos_table[positions[t]]), written as float (the residual stream).
// Reference: kelpie-models/kelpie_models/models/torch/gpt2.py:90.
template <typename W>
__global__ void embed_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ positions,
                             const W* __restrict__ table, const W* __restrict__ pos_table,
                             float* __restrict__ out, int width, int n_vocab, int n_positions) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  int t = blockIdx.x;
  int id = ids[t];
  id = id < 0 ? 0 : (id >= n_vocab ? n_vocab - 1 : id);  // ids are validated on the host
  const W* row = table + size_t(id) * width;
  const W* prow = nullptr;
  if (pos_table != nullptr) {
    int p = positions[t];
    p = p < 0 ? 0 : (p >= n_positions ? n_positions - 1 : p);
    prow = pos_table + size_t(p) * width;
  }
  float* o = out + size_t(t) * width;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float v = to_float(row[d]);
    if (prow != nullptr) v += to_float(prow[d]);
    o[d] = v;
  }
}

extern "C" int r2_embed(const int32_t* ids, const int32_t* positions, const void* table, const void* pos_table,
                        float* out, int n_rows, int width, int n_vocab, int n_positions, int wdtype,
                        cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (width < 1 || n_vocab < 1) return R2_BAD_SHAPE;
  int threads = width >= 256 ? 256 : (width >= 128 ? 128 : 64);
  if (wdtype == R2_F32) {
    r2_launch(embed_kernel<float>, dim3(n_rows), dim3(threads), size_t(0), stream, ids, positions, (const float*)table, (const float*)pos_table,
                                                        out, width, n_vocab, n_positions);
  } else if (wdtype == R2_BF16) {
    r2_launch(embed_kernel<bf16>, dim3(n_rows), dim3(threads), size_t(0), stream, ids, positions, (const bf16*)table, (const bf16*)pos_table,
                                                       out, width, n_vocab, n_positions);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// ---------------------------------------------------------------------------------------------
// y = (x - mean) / sqrt(var + eps) * gamma + beta, biased variance, statistics in float.
// `rows` (may be null) picks the input rows: output row i reads input row rows[i].
// Reference: kelpie-models/kelpie_models/kernels/ops/layer_norm.py:21-23.
template <typename O>
__global__ void layer_norm_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows,
                                  const float* __restrict__ gamma, const float* __restrict__ beta,
                                  O* __restrict__ out, int width, float eps) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  extern __shared__ float row_s[];
  __shared__ float scratch[33];
  int r = blockIdx.x;
  int src = rows != nullptr ? rows[r] : r;
  const float* xr = x + size_t(src) * width;
  float sum = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float v = xr[d];
    row_s[d] = v;
    sum += v;
  }
  float mean = block_sum(sum, scratch) / float(width);
  float sq = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float c = row_s[d] - mean;
    sq += c * c;
  }
  float var = block_sum(sq, scratch) / float(width);
  float inv = 1.f / sqrtf(var + eps);
  O* o = out + size_t(r) * width;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    o[d] = from_float<O>((row_s[d] - mean) * inv * gamma[d] + beta[d]);
  }
}

// The same with one warp per row, the row in registers, no block-wide barrier: rows of up to
// 2,048 elements whose length is a multiple of 4 (wider or unaligned rows take the kernel above).
template <typename O>
__global__ void __launch_bounds__(128)
layer_norm_warp_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, const float* __restrict__ gamma,
                       const float* __restrict__ beta, O* __restrict__ out, int n_rows, int width, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (r >= n_rows) return;
  const int src = rows != nullptr ? rows[r] : r;
  const float4* xr = reinterpret_cast<const float4*>(x + size_t(src) * width);
  constexpr int CHUNKS = 2048 / 128;
  float4 v[CHUNKS];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    int k = (lane + 32 * i) * 4;
    v[i] = k < width ? xr[lane + 32 * i] : make_float4(0.f, 0.f, 0.f, 0.f);
    sum += v[i].x + v[i].y + v[i].z + v[i].w;
  }
  const float mean = warp_sum(sum) / float(width);
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    int k = (lane + 32 * i) * 4;
    if (k < width) {
      float a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
      sq += a * a + b * b + c * c + d * d;
    }
  }
  const float inv = 1.f / sqrtf(warp_sum(sq) / float(width) + eps);
  O* o = out + size_t(r) * width;
#pragma unroll
  for (int i = 0; i < CHUNKS; ++i) {
    int k = (lane + 32 * i) * 4;
    if (k < width) {
      float4 g = *reinterpret_cast<const float4*>(gamma + k);
      float4 b = *reinterpret_cast<const float4*>(beta + k);
      const float y0 = (v[i].x - mean) * inv * g.x + b.x, y1 = (v[i].y - mean) * inv * g.y + b.y;
      const float y2 = (v[i].z - mean) * inv * g.z + b.z, y3 = (v[i].w - mean) * inv * g.w + b.w;
      if constexpr (sizeof(O) == 2) {  // four values, one 8-byte store (rows are multiples of 4 wide and the output 8-byte aligned)
        __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
        *reinterpret_cast<uint2*>(o + k) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
      } else {
        *reinterpret_cast<float4*>(o + k) = make_float4(y0, y1, y2, y3);
      }
    }
  }
}

extern "C" int r2_layer_norm(const float* x, const int32_t* rows, const float* gamma, const float* beta, void* out,
                             int n_rows, int width, float eps, int odtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (width < 1 || size_t(width) * 4 > 200 * 1024) return R2_BAD_SHAPE;
  const bool aligned = width % 4 == 0 && !(reinterpret_cast<uintptr_t>(x) & 15) && !(reinterpret_cast<uintptr_t>(gamma) & 15) &&
                       !(reinterpret_cast<uintptr_t>(beta) & 15) && !(reinterpret_cast<uintptr_t>(out) & 15);
  if (width <= 2048 && aligned && (odtype == R2_F32 || odtype == R2_BF16)) {
    dim3 grid((n_rows + 3) / 4);
    if (odtype == R2_F32) {
      r2_launch(layer_norm_warp_kernel<float>, grid, dim3(128), size_t(0), stream, x, rows, gamma, beta, (float*)out, n_rows, width, eps);
    } else {
      r2_launch(layer_norm_warp_kernel<bf16>, grid, dim3(128), size_t(0), stream, x, rows, gamma, beta, (bf16*)out, n_rows, width, eps);
    }
    return launch_status();
  }
  int threads = width >= 1024 ? 256 : 128;
  size_t smem = size_t(width) * sizeof(float);
  if (odtype == R2_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(layer_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    r2_launch(layer_norm_kernel<float>, dim3(n_rows), dim3(threads), size_t(smem), stream, x, rows, gamma, beta, (float*)out, width, eps);
  } else if (odtype == R2_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(layer_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    r2_launch(layer_norm_kernel<bf16>, dim3(n_rows), dim3(threads), size_t(smem), stream, x, rows, gamma, beta, (bf16*)out, width, eps);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}

// ---------------------------------------------------------------------------------------------
// Keys and values of this step's rows go to their cache slots before attention reads them
// (kelpie-models/kelpie_models/kernels/ops/paged_attention.py:44-53). A slot is
// page * page_size + offset; inside a page the layout is [kv_head][offset][head_dim], and a
// page of this layer starts every `page_stride` elements.
template <typename A, typename C>
__global__ void kv_write_kernel(const A* __restrict__ k_src, const A* __restrict__ v_src, int src_row_stride,
                                C* __restrict__ k_cache, C* __restrict__ v_cache,
                                const int32_t* __restrict__ slot_mapping, int n_kv_heads, int head_dim,
                                int page_size, long long page_stride, int n_pages) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  int t = blockIdx.x;
  int slot = slot_mapping[t];
  int page = slot / page_size, off = slot % page_size;
  if (slot < 0 || page >= n_pages) return;  // slots are validated on the host; never write outside the pool
  int width = n_kv_heads * head_dim;
  const A* ks = k_src + size_t(t) * src_row_stride;
  const A* vs = v_src + size_t(t) * src_row_stride;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    int h = i / head_dim, d = i % head_dim;
    size_t dst = size_t(page) * page_stride + (size_t(h) * page_size + off) * head_dim + d;
    k_cache[dst] = from_float<C>(to_float(ks[i]));
    v_cache[dst] = from_float<C>(to_float(vs[i]));
  }
}

extern "C" int r2_kv_write(const void* k_src, const void* v_src, int src_row_stride, void* k_cache, void* v_cache,
                           const int32_t* slot_mapping, int n_rows, int n_kv_heads, int head_dim, int page_size,
                           long long page_stride, int n_pages_total, int dtype, cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (n_kv_heads < 1 || head_dim < 1 || page_size < 1 || n_pages_total < 1) return R2_BAD_SHAPE;
  int width = n_kv_heads * head_dim;
  int threads = width >= 256 ? 256 : 128;
  if (dtype == R2_F32) {
    r2_launch(kv_write_kernel<float, float>, dim3(n_rows), dim3(threads), size_t(0), stream, (const float*)k_src, (const float*)v_src, src_row_stride,
                                                                  (float*)k_cache, (float*)v_cache, slot_mapping,
                                                                  n_kv_heads, head_dim, page_size, page_stride, n_pages_total);
  } else if (dtype == R2_BF16) {
    r2_launch(kv_write_kernel<bf16, bf16>, dim3(n_rows), dim3(threads), size_t(0), stream, (const bf16*)k_src, (const bf16*)v_src, src_row_stride,
                                                                (bf16*)k_cache, (bf16*)v_cache, slot_mapping,
                                                                n_kv_heads, head_dim, page_size, page_stride, n_pages_total);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}
