// The boundary between two layers of a block that runs its mixer and its feed-forward side by side on
// the same input, gates each result, and hands on a weighted average of all layer results so far;
// and the two norms (Dynamic Tanh) that the next layer reads. One pass over the row does all of it:
//
//   s      = x + sum_k sigmoid(gate_k) * delta_k            (k < 2; a null gate means a plain add)
//   X[n]   = s                                              (the layer's result joins the history)
//   z      = sum_{j <= n} mix[j] * X[j]                     (null mix: z = s)
//   y_k    = tanh(alpha_k * z) * w_k + b_k                  (k < 2: the norms of the next layer, or the
//                                                            model's last norm on the wanted rows)
//
// x, X, z and all sums are float32. With `row_map` only those rows are worked out (the rows whose
// logits are wanted) and nothing is stored but y: the history is read, not extended.
// Also here: the feed-forward's activation xIELU.
#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ float4 ld4(const void* p, int dtype, size_t i) {   // i % 4 == 0
  if (dtype == HB_DTYPE_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
  const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
  return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                     __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}
__device__ __forceinline__ float ld1(const void* p, int dtype, size_t i) {
  return dtype == HB_DTYPE_F32 ? reinterpret_cast<const float*>(p)[i]
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void st4(void* p, int dtype, size_t i, float4 v) {
  if (dtype == HB_DTYPE_F32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + i) = v;
  } else {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<unsigned*>(&a);
    raw.y = *reinterpret_cast<unsigned*>(&b);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p) + i) = raw;
  }
}
__device__ __forceinline__ void st1(void* p, int dtype, size_t i, float v) {
  if (dtype == HB_DTYPE_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float sigmoidf(float v) { return 1.f / (1.f + expf(-v)); }

struct BoundaryArgs {
  const float* x;            // [N, W] the layer's input
  const void* delta[2];      // [N, W] sub-layer results (or null)
  const void* gate[2];       // [N, W] what the sigmoid takes (or null: factor 1)
  int delta_dtype[2], gate_dtype[2];
  float* hist;               // [entries, N, W] results of the layers so far, X[0] first (or null)
  long long hist_stride;     // N * W
  int n_prev;                // entries of the history that are filled
  const float* mix;          // [n_prev + 1] (or null)
  float* z_out;              // [rows, W] (or null)
  const float* alpha[2];     // one float each
  const void* w[2];          // [W]
  const void* b[2];          // [W]
  int wb_dtype;
  void* y[2];                // [rows, W]
  int y_dtype;
  const int* row_map;
  int width;
};

// VEC elements from index i (i % VEC == 0) as floats.
template <int VEC>
__device__ __forceinline__ void ldv(const void* p, int dtype, size_t i, float (&v)[VEC]) {
  if constexpr (VEC == 4) {
    const float4 q = ld4(p, dtype, i);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  } else {
    v[0] = ld1(p, dtype, i);
  }
}
template <int VEC>
__device__ __forceinline__ void stv(void* p, int dtype, size_t i, const float (&v)[VEC]) {
  if constexpr (VEC == 4) st4(p, dtype, i, make_float4(v[0], v[1], v[2], v[3]));
  else st1(p, dtype, i, v[0]);
}

// VEC = 4: width % 4 == 0, 16-byte accesses; VEC = 1: any width.
template <int VEC>
__global__ void boundary_kernel(const BoundaryArgs a) {
  const int r = blockIdx.x;
  const size_t src = a.row_map ? (size_t)a.row_map[r] : (size_t)r;
  const float alpha[2] = {a.y[0] ? *a.alpha[0] : 0.f, a.y[1] ? *a.alpha[1] : 0.f};
  for (int j = (blockIdx.y * blockDim.x + threadIdx.x) * VEC; j < a.width; j += gridDim.y * blockDim.x * VEC) {
    const size_t at = src * a.width + j;
    float s[VEC], add[VEC];
    ldv<VEC>(a.x, HB_DTYPE_F32, at, s);
#pragma unroll
    for (int e = 0; e < VEC; ++e) add[e] = 0.f;
    // the gated results are summed first, then added to the stream
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (!a.delta[k]) continue;
      float d[VEC];
      ldv<VEC>(a.delta[k], a.delta_dtype[k], at, d);
      if (a.gate[k]) {
        float g[VEC];
        ldv<VEC>(a.gate[k], a.gate_dtype[k], at, g);
#pragma unroll
        for (int e = 0; e < VEC; ++e) d[e] *= sigmoidf(g[e]);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) add[e] += d[e];
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) s[e] += add[e];
    float z[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) z[e] = s[e];
    if (a.hist) {
      if (!a.row_map) stv<VEC>(a.hist + (size_t)a.n_prev * a.hist_stride, HB_DTYPE_F32, at, s);
      if (a.mix) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) z[e] = 0.f;
        for (int p = 0; p < a.n_prev; ++p) {          // in the order of the layers, the new result last
          const float m = a.mix[p];
          float h[VEC];
          ldv<VEC>(a.hist + (size_t)p * a.hist_stride, HB_DTYPE_F32, at, h);
#pragma unroll
          for (int e = 0; e < VEC; ++e) z[e] += m * h[e];
        }
        const float m = a.mix[a.n_prev];
#pragma unroll
        for (int e = 0; e < VEC; ++e) z[e] += m * s[e];
      }
    }
    const size_t to = (size_t)r * a.width + j;
    if (a.z_out) stv<VEC>(a.z_out, HB_DTYPE_F32, to, z);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (!a.y[k]) continue;
      float y[VEC], w[VEC], b[VEC];
      ldv<VEC>(a.w[k], a.wb_dtype, j, w);
      ldv<VEC>(a.b[k], a.wb_dtype, j, b);
#pragma unroll
      for (int e = 0; e < VEC; ++e) y[e] = tanhf(alpha[k] * z[e]) * w[e] + b[e];
      stv<VEC>(a.y[k], a.y_dtype, to, y);
    }
  }
}

// z > 0: ap z^2 + z/2;  z <= 0: an (e^z - 1 - z) + z/2;  coef = (ap, an), float32
__device__ __forceinline__ float xielu1(float z, float ap, float an) {
  return z > 0.f ? ap * z * z + 0.5f * z : an * (expm1f(z) - z) + 0.5f * z;
}

template <typename T>
__global__ void xielu_kernel(const T* __restrict__ in, T* __restrict__ out, const float* __restrict__ coef,
                             long long n) {
  const float ap = coef[0], an = coef[1];
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float z = hb::to_f32(in[i]);
    out[i] = hb::from_f32<T>(xielu1(z, ap, an));
  }
}

// bfloat16, n % 8 == 0: eight elements a thread, 16-byte accesses
__global__ void xielu_bf16x8_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                    const float* __restrict__ coef, long long n8) {
  const float ap = coef[0], an = coef[1];
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const uint4 raw = in[i];
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t r[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float lo = xielu1(__uint_as_float(w[e] << 16), ap, an);
      const float hi = xielu1(__uint_as_float(w[e] & 0xffff0000u), ap, an);
      const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
      r[e] = *reinterpret_cast<const uint32_t*>(&p);
    }
    out[i] = make_uint4(r[0], r[1], r[2], r[3]);
  }
}

}  // namespace

extern "C" int hb_gated_depth_dyt(const float* x, const void* delta0, int delta0_dtype, const void* gate0, int gate0_dtype,
                                  const void* delta1, int delta1_dtype, const void* gate1, int gate1_dtype,
                                  float* hist, long long hist_stride, int n_prev, const float* mix, float* z_out,
                                  const float* alpha0, const void* w0, const void* b0, void* y0,
                                  const float* alpha1, const void* w1, const void* b1, void* y1,
                                  int wb_dtype, int y_dtype, const int* row_map, int rows, int width,
                                  cudaStream_t stream) {
  if (!x || rows < 0 || width <= 0 || n_prev < 0) return HB_ERR_BAD_ARG;
  if ((y0 && (!alpha0 || !w0 || !b0)) || (y1 && (!alpha1 || !w1 || !b1))) return HB_ERR_BAD_ARG;
  if (mix && !hist) return HB_ERR_BAD_ARG;
  if (rows == 0) return HB_OK;
  BoundaryArgs a;
  a.x = x;
  a.delta[0] = delta0; a.delta[1] = delta1; a.gate[0] = gate0; a.gate[1] = gate1;
  a.delta_dtype[0] = delta0_dtype; a.delta_dtype[1] = delta1_dtype;
  a.gate_dtype[0] = gate0_dtype; a.gate_dtype[1] = gate1_dtype;
  a.hist = hist; a.hist_stride = hist_stride; a.n_prev = n_prev; a.mix = mix; a.z_out = z_out;
  a.alpha[0] = alpha0; a.alpha[1] = alpha1; a.w[0] = w0; a.w[1] = w1; a.b[0] = b0; a.b[1] = b1;
  a.wb_dtype = wb_dtype; a.y[0] = y0; a.y[1] = y1; a.y_dtype = y_dtype; a.row_map = row_map; a.width = width;
  const int threads = 128;
  if (width % 4 == 0) {
    const int per_row = (width / 4 + threads - 1) / threads;
    dim3 grid(rows, per_row > 8 ? 8 : per_row);
    boundary_kernel<4><<<grid, threads, 0, stream>>>(a);
  } else {
    const int per_row = (width + threads - 1) / threads;
    dim3 grid(rows, per_row > 8 ? 8 : per_row);
    boundary_kernel<1><<<grid, threads, 0, stream>>>(a);
  }
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_xielu(const void* in, void* out, int dtype, const float* coef, long long n, cudaStream_t stream) {
  if (!in || !out || !coef || n < 0) return HB_ERR_BAD_ARG;
  if (n == 0) return HB_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (dtype == HB_DTYPE_F32)
    xielu_kernel<float><<<(int)blocks, 256, 0, stream>>>((const float*)in, (float*)out, coef, n);
  else if (dtype == HB_DTYPE_BF16 && n % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    long long b8 = (n / 8 + 255) / 256;
    if (b8 > 148 * 16) b8 = 148 * 16;
    xielu_bf16x8_kernel<<<(int)b8, 256, 0, stream>>>((const uint4*)in, (uint4*)out, coef, n / 8);
  } else if (dtype == HB_DTYPE_BF16)
    xielu_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, coef, n);
  else
    return HB_ERR_BAD_ARG;
  HB_LAUNCH_CHECK();
  return HB_OK;
}
