// Latent attention's own small steps. The cache of such a mixer holds one latent row per token, from
// which every head's keys and values are linear maps; attention itself runs on the latents with the
// key map folded into the query and the value map applied to the result, through the paged attention
// kernels (one shared "kv head" whose keys and values are the same rows).
//
//   latent_append:  c = x / sqrt(mean(x^2) + eps) * w  (float32), written to the token's place in its page,
//                   zero-filled up to the page's row length
//   head_gate:      out[t, h, :] = in[t, h, :] * sigmoid(g[t, h])
#include "api.h"
#include "common.cuh"

namespace {

template <typename T>
__global__ void latent_append_kernel(const T* __restrict__ in, long long in_stride, const T* __restrict__ w, float eps,
                                     const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                     const int* __restrict__ block_table, int table_stride, T* __restrict__ pages,
                                     int page_size, int rank, int row_len) {
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const T* row = in + (size_t)t * in_stride;
  float ss = 0.f;
  for (int j = threadIdx.x; j < rank; j += blockDim.x) {
    const float v = hb::to_f32(row[j]);
    ss += v * v;
  }
  const float inv = rsqrtf(hb::block_sum(ss, scratch) / (float)rank + eps);
  const int pos = positions[t];
  const int page = block_table[(size_t)seq_of_token[t] * table_stride + pos / page_size];
  if (page < 0) return;
  T* dst = pages + ((size_t)page * page_size + (pos % page_size)) * row_len;
  for (int j = threadIdx.x; j < row_len; j += blockDim.x)
    dst[j] = j < rank ? hb::from_f32<T>(hb::to_f32(row[j]) * inv * hb::to_f32(w[j])) : hb::from_f32<T>(0.f);
}

template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ in, const T* __restrict__ gate, long long gate_stride,
                                 T* __restrict__ out, int heads, int dim) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < heads * dim; i += blockDim.x) {
    const int h = i / dim;
    const float g = hb::to_f32(gate[(size_t)t * gate_stride + h]);
    const size_t at = (size_t)t * heads * dim + i;
    out[at] = hb::from_f32<T>(hb::to_f32(in[at]) / (1.f + expf(-g)));
  }
}

}  // namespace

extern "C" int hb_latent_append(const void* in, int dtype, long long in_stride, const void* w, float eps,
                                const int* positions, const int* seq_of_token, const int* block_table,
                                int table_stride, void* pages, int page_size, int rank, int row_len, int n_tokens,
                                cudaStream_t stream) {
  if (!in || !w || !positions || !seq_of_token || !block_table || !pages) return HB_ERR_BAD_ARG;
  if (rank <= 0 || row_len < rank || page_size <= 0 || table_stride <= 0 || n_tokens < 0 || in_stride < rank)
    return HB_ERR_BAD_ARG;
  if (n_tokens == 0) return HB_OK;
  const int threads = rank >= 256 ? 256 : (rank >= 128 ? 128 : 64);
  if (dtype == HB_DTYPE_F32)
    latent_append_kernel<float><<<n_tokens, threads, 0, stream>>>(
        (const float*)in, in_stride, (const float*)w, eps, positions, seq_of_token, block_table, table_stride,
        (float*)pages, page_size, rank, row_len);
  else if (dtype == HB_DTYPE_BF16)
    latent_append_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        (const __nv_bfloat16*)in, in_stride, (const __nv_bfloat16*)w, eps, positions, seq_of_token, block_table,
        table_stride, (__nv_bfloat16*)pages, page_size, rank, row_len);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_head_gate(const void* in, const void* gate, long long gate_stride, void* out, int dtype,
                            int n_tokens, int heads, int dim, cudaStream_t stream) {
  if (!in || !gate || !out || heads <= 0 || dim <= 0 || n_tokens < 0 || gate_stride < heads) return HB_ERR_BAD_ARG;
  if (n_tokens == 0) return HB_OK;
  const int threads = heads * dim >= 256 ? 256 : 128;
  if (dtype == HB_DTYPE_F32)
    head_gate_kernel<float><<<n_tokens, threads, 0, stream>>>((const float*)in, (const float*)gate, gate_stride,
                                                              (float*)out, heads, dim);
  else if (dtype == HB_DTYPE_BF16)
    head_gate_kernel<__nv_bfloat16><<<n_tokens, threads, 0, stream>>>(
        (const __nv_bfloat16*)in, (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, heads, dim);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  return HB_OK;
}
