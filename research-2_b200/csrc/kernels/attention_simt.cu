// Paged causal attention on the CUDA cores, all arithmetic in float: the true 32-bit path, and
// the general path of the bfloat16 engine for head sizes or batches the tensor-core kernels refuse.
//
// One warp computes one (row, head): it walks the row's visible keys in position order in tiles
// of 32 (lane = key), keeps a running maximum and sum (online softmax) and accumulates P.V with
// lanes over the head dimension. The walk depends only on the row's position, its window and
// the head size, never on how the step was cut or batched, so a row's output is the same bits
// whichever batch it came in.
//
// Reference formulas: kelpie-models/kelpie_models/kernels/ops/paged_attention.py:160-240
// (scores * scale 179, visibility 186-212, softmax 215-240, PV 182-183, pad rows zero 140).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HEAD_DIM = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, int q_row_stride, T* __restrict__ out, int out_row_stride,
                      const T* __restrict__ k_cache, const T* __restrict__ v_cache, long long page_stride,
                      int page_size, const int32_t* __restrict__ block_tables, int table_width,
                      const int32_t* __restrict__ row_entry, const int32_t* __restrict__ positions,
                      const int32_t* __restrict__ seq_lens, int n_heads, int n_kv_heads, int head_dim,
                      float scale, int window, int n_pages) {
  pdl_launch_dependents();  // the next kernel may begin its prologue
  pdl_wait();               // the previous kernel's writes are visible from here on
  __shared__ float q_s[WARPS][MAX_HEAD_DIM];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * WARPS + warp;
  if (h >= n_heads) return;
  T* o = out + size_t(t) * out_row_stride + size_t(h) * head_dim;
  const int e = row_entry[t];
  if (e < 0) {  // a pad row
    for (int d = lane; d < head_dim; d += 32) o[d] = from_float<T>(0.f);
    return;
  }
  const int pos = positions[t];
  const int seq_len = seq_lens[e];
  const int kvh = h / (n_heads / n_kv_heads);
  const int32_t* table = block_tables + size_t(e) * table_width;
  const T* qr = q + size_t(t) * q_row_stride + size_t(h) * head_dim;
  for (int d = lane; d < head_dim; d += 32) q_s[warp][d] = to_float(qr[d]);
  __syncwarp();

  int last = pos < seq_len - 1 ? pos : seq_len - 1;       // newest visible key
  int first = window > 0 ? (pos - window + 1 > 0 ? pos - window + 1 : 0) : 0;
  float m = -INFINITY, l = 0.f;
  float acc[MAX_HEAD_DIM / 32];
#pragma unroll
  for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) acc[i] = 0.f;
  const size_t head_off = size_t(kvh) * page_size * head_dim;

  for (int j0 = first; j0 <= last; j0 += 32) {
    int j = j0 + lane;
    bool valid = j <= last;
    float s = -INFINITY;
    if (valid) {
      int page = table[j / page_size];
      page = (page < 0 || page >= n_pages) ? 0 : page;
      const T* kr = k_cache + size_t(page) * page_stride + head_off + size_t(j % page_size) * head_dim;
      float dot = 0.f;
      for (int d = 0; d < head_dim; ++d) dot = fmaf(q_s[warp][d], to_float(kr[d]), dot);
      s = dot * scale;
    }
    float m_new = fmaxf(m, warp_max(s));
    float corr = expf(m - m_new);  // exp(-inf) = 0 on the first tile
    float p = valid ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) acc[i] *= corr;
    int n_valid = last - j0 + 1 < 32 ? last - j0 + 1 : 32;
    for (int jj = 0; jj < n_valid; ++jj) {
      float pj = __shfl_sync(0xffffffffu, p, jj);
      int key = j0 + jj;
      int page = table[key / page_size];
      page = (page < 0 || page >= n_pages) ? 0 : page;
      const T* vr = v_cache + size_t(page) * page_stride + head_off + size_t(key % page_size) * head_dim;
#pragma unroll
      for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) {
        int d = lane + 32 * i;
        if (d < head_dim) acc[i] = fmaf(pj, to_float(vr[d]), acc[i]);
      }
    }
  }
  float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int i = 0; i < MAX_HEAD_DIM / 32; ++i) {
    int d = lane + 32 * i;
    if (d < head_dim) o[d] = from_float<T>(acc[i] * inv);
  }
}

}  // namespace

// q [T, n_heads * head_dim] with row stride q_row_stride (it may be a slice of a fused qkv
// buffer), out [T, n_heads * head_dim]; the cache of this layer as in r2_kv_write.
extern "C" int r2_attention_simt(const void* q, int q_row_stride, void* out, int out_row_stride, const void* k_cache,
                                 const void* v_cache, long long page_stride, int page_size,
                                 const int32_t* block_tables, int table_width, const int32_t* row_entry,
                                 const int32_t* positions, const int32_t* seq_lens, int n_rows, int n_heads,
                                 int n_kv_heads, int head_dim, float scale, int window, int n_pages, int dtype,
                                 cudaStream_t stream) {
  if (n_rows <= 0) return R2_OK;
  if (head_dim < 1 || head_dim > MAX_HEAD_DIM) return R2_UNSUPPORTED;
  if (n_heads < 1 || n_kv_heads < 1 || n_heads % n_kv_heads != 0 || page_size < 1 || window < 0) return R2_BAD_SHAPE;
  dim3 grid(n_rows, (n_heads + WARPS - 1) / WARPS);
  if (dtype == R2_F32) {
    r2_launch(attention_simt_kernel<float>, dim3(grid), dim3(WARPS * 32), size_t(0), stream, 
        (const float*)q, q_row_stride, (float*)out, out_row_stride, (const float*)k_cache, (const float*)v_cache,
        page_stride, page_size, block_tables, table_width, row_entry, positions, seq_lens, n_heads, n_kv_heads,
        head_dim, scale, window, n_pages);
  } else if (dtype == R2_BF16) {
    r2_launch(attention_simt_kernel<bf16>, dim3(grid), dim3(WARPS * 32), size_t(0), stream, 
        (const bf16*)q, q_row_stride, (bf16*)out, out_row_stride, (const bf16*)k_cache, (const bf16*)v_cache,
        page_stride, page_size, block_tables, table_width, row_entry, positions, seq_lens, n_heads, n_kv_heads,
        head_dim, scale, window, n_pages);
  } else {
    return R2_BAD_DTYPE;
  }
  return launch_status();
}
