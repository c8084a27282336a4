// The matrix memory of the mLSTM: per head a matrix S [dim, vdim], a vector n [dim] and a running
// maximum m that every token updates and reads,
//   i = cap tanh((z_i + b_i) / cap),  f = logsigmoid(cap tanh((z_f + b_f) / cap))
//   m' = max(f + m, i);  S' = e^(f + m - m') S + e^(i - m') k v^T;  n' = e^(f + m - m') n + e^(i - m') k
//   o = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6)
// in three kernels, all float32:
//   mlstm_gates       the gates' logarithms for all tokens side by side, the scan of m token after token (adds and
//                     maxima only), then keep = e^(f + m - m'), take = e^(i - m') and floor = e^(-m') side by side
//   mlstm_recurrence  S and n token after token. n is one more column of S whose value is always 1, so that
//                     n' . q falls out as one more output. A column lives in the registers of L lanes, R rows each.
//   mlstm_out_norm    the division, the RMS norm of every head's output, the weight and the sigmoid gate
// A request's state is one float32 row: [heads][vdim + 1][dim] (column-major S, then n), then m [heads]. It
// starts at zero, m too.
#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ float load_el(const void* p, int dtype, size_t i) {
  return dtype == HB_DTYPE_F32 ? reinterpret_cast<const float*>(p)[i]
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

constexpr int GATE_THREADS = 128;

// grid (heads, sequences). z [N, 2 * heads] float32: the input gates' pre-activations, then the forget gates'.
__global__ void __launch_bounds__(GATE_THREADS)
mlstm_gates_kernel(const float* __restrict__ z, const float* __restrict__ bias_i, const float* __restrict__ bias_f,
                   float cap, float* __restrict__ state, long long state_stride, long long m_off,
                   const int* __restrict__ cu_seqlens, const int* __restrict__ slots, float* __restrict__ keep,
                   float* __restrict__ take, float* __restrict__ floor_, int heads) {
  __shared__ float warp_f[GATE_THREADS / 32], warp_i[GATE_THREADS / 32], carry[GATE_THREADS / 32 + 1];
  const int h = blockIdx.x, seq = blockIdx.y;
  const int begin = cu_seqlens[seq], end = cu_seqlens[seq + 1];
  if (begin >= end) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* m_state = state + (size_t)slots[seq] * state_stride + m_off + h;
  const float bi = bias_i ? bias_i[h] : 0.f, bf = bias_f ? bias_f[h] : 0.f;
  const float inv_cap = 1.f / cap;
  float m_before_block = *m_state;          // every thread carries the maximum that enters the block of tokens
  // A token maps the maximum m to max(m + f, i); two tokens in turn map it to max(m + f1 + f2, max(i1 + f2, i2)):
  // the pairs (F, I) combine associatively, so a block of tokens is scanned in a few steps instead of one by one.
  for (int t0 = begin; t0 < end; t0 += GATE_THREADS) {
    const int t = t0 + threadIdx.x;
    float gi = -INFINITY, gf = 0.f;          // past the end: the identity map
    if (t < end) {
      const float zi = z[(size_t)t * 2 * heads + h] + bi, zf = z[(size_t)t * 2 * heads + heads + h] + bf;
      const float cf = cap * tanhf(zf * inv_cap);
      gi = cap * tanhf(zi * inv_cap);
      gf = fminf(cf, 0.f) - log1pf(expf(-fabsf(cf)));      // log sigmoid
    }
    float F = gf, I = gi;                    // inclusive scan over the warp's tokens
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float Fp = __shfl_up_sync(0xffffffffu, F, off), Ip = __shfl_up_sync(0xffffffffu, I, off);
      if (lane >= off) {
        I = fmaxf(Ip + F, I);
        F = Fp + F;
      }
    }
    if (lane == 31) { warp_f[warp] = F; warp_i[warp] = I; }
    __syncthreads();
    if (threadIdx.x == 0) {                  // the maximum that enters each warp's tokens, and the next block's
      float m = m_before_block;
      for (int w2 = 0; w2 < GATE_THREADS / 32; ++w2) {
        carry[w2] = m;
        m = fmaxf(m + warp_f[w2], warp_i[w2]);
      }
      carry[GATE_THREADS / 32] = m;
    }
    __syncthreads();
    const float now = fmaxf(carry[warp] + F, I);
    float before = __shfl_up_sync(0xffffffffu, now, 1);
    if (lane == 0) before = carry[warp];
    if (t < end) {
      keep[(size_t)t * heads + h] = expf(gf + before - now);
      take[(size_t)t * heads + h] = expf(gi - now);
      floor_[(size_t)t * heads + h] = expf(-now);
    }
    m_before_block = carry[GATE_THREADS / 32];
    __syncthreads();
  }
  if (threadIdx.x == 0) *m_state = m_before_block;
}

constexpr int REC_THREADS = 256;
constexpr int REC_TOKENS = 8;      // tokens staged in shared memory at a time

// grid (column groups, heads, sequences); a block holds REC_THREADS / L columns of one head's S (column vdim is n).
// Lane l of a column's L lanes holds rows l * R .. l * R + R - 1. Rows past dim hold zeros and meet zeros.
template <int R>
__global__ void __launch_bounds__(REC_THREADS)
mlstm_recurrence_kernel(const void* __restrict__ proj, int proj_dtype, long long ld, int q_off, int k_off, int v_off,
                        float q_scale, const float* __restrict__ keep, const float* __restrict__ take,
                        float* __restrict__ state, long long state_stride, const int* __restrict__ cu_seqlens,
                        const int* __restrict__ slots, float* __restrict__ o, float* __restrict__ nq, int heads,
                        int dim, int vdim, int L) {
  extern __shared__ float sm[];       // per staged token: q [dim_pad], k [dim_pad], v [cols], keep, take
  const int h = blockIdx.y, seq = blockIdx.z;
  const int begin = cu_seqlens[seq], end = cu_seqlens[seq + 1];
  if (begin >= end) return;
  const int cols_per_block = REC_THREADS / L;
  const int dim_pad = L * R;
  const int col0 = blockIdx.x * cols_per_block;
  const int col = col0 + threadIdx.x / L;          // my column; vdim = the column of n
  const int sub = threadIdx.x % L;
  const bool live = col <= vdim;
  const int per_token = 2 * dim_pad + cols_per_block + 2;
  float* S_col = state + (size_t)slots[seq] * state_stride + ((size_t)h * (vdim + 1) + (live ? col : 0)) * dim;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = sub * R + r;
    S[r] = (live && d < dim) ? S_col[d] : 0.f;
  }
  for (int t0 = begin; t0 < end; t0 += REC_TOKENS) {
    const int count = min(REC_TOKENS, end - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < count * dim_pad; i += REC_THREADS) {
      const int j = i / dim_pad, d = i - j * dim_pad;
      const size_t row = (size_t)(t0 + j) * ld + (size_t)h * dim + d;
      float* dst = sm + j * per_token;
      dst[d] = d < dim ? load_el(proj, proj_dtype, row + q_off) * q_scale : 0.f;
      dst[dim_pad + d] = d < dim ? load_el(proj, proj_dtype, row + k_off) : 0.f;
    }
    for (int i = threadIdx.x; i < count * (cols_per_block + 2); i += REC_THREADS) {
      const int j = i / (cols_per_block + 2), c = i - j * (cols_per_block + 2);
      float* dst = sm + j * per_token + 2 * dim_pad;
      if (c < cols_per_block) {
        const int cc = col0 + c;
        dst[c] = cc < vdim ? load_el(proj, proj_dtype, (size_t)(t0 + j) * ld + v_off + (size_t)h * vdim + cc)
                           : (cc == vdim ? 1.f : 0.f);
      } else {
        dst[c] = (c == cols_per_block ? keep : take)[(size_t)(t0 + j) * heads + h];
      }
    }
    __syncthreads();
    for (int j = 0; j < count; ++j) {
      const float* tok = sm + j * per_token;
      const float* qs = tok + sub * R;
      const float* ks = tok + dim_pad + sub * R;
      const float a = tok[2 * dim_pad + cols_per_block];
      const float bv = tok[2 * dim_pad + cols_per_block + 1] * tok[2 * dim_pad + threadIdx.x / L];
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        S[r] = fmaf(bv, ks[r], a * S[r]);
        acc = fmaf(S[r], qs[r], acc);
      }
      for (int off = L >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (sub == 0 && live) {
        if (col < vdim) o[((size_t)(t0 + j) * heads + h) * vdim + col] = acc;
        else nq[(size_t)(t0 + j) * heads + h] = acc;
      }
    }
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = sub * R + r;
      if (d < dim) S_col[d] = S[r];
    }
  }
}

// The same recurrence for sizes whose rows are whole 16-byte runs (the usual case): q, k and v of the next
// REC_AHEAD tokens come into shared memory with cp.async, as they are stored, while the block works on the
// tokens before them; nothing waits for global memory between tokens. T is the projection's element type.
constexpr int REC_AHEAD = 32;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_4(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(raw.x << 16); v[1] = __uint_as_float(raw.x & 0xffff0000u);
  v[2] = __uint_as_float(raw.y << 16); v[3] = __uint_as_float(raw.y & 0xffff0000u);
}

// R consecutive elements as floats, by the widest loads their size allows (16 bytes where R elements fill them)
template <int R>
__device__ __forceinline__ void load_row(const float* p, float (&v)[R]) {
#pragma unroll
  for (int r = 0; r < R; r += 4) {
    const float4 a = *reinterpret_cast<const float4*>(p + r);
    v[r] = a.x; v[r + 1] = a.y; v[r + 2] = a.z; v[r + 3] = a.w;
  }
}
template <int R>
__device__ __forceinline__ void load_row(const __nv_bfloat16* p, float (&v)[R]) {
  if constexpr (R % 8 == 0) {
#pragma unroll
    for (int r = 0; r < R; r += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(p + r);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[r + 2 * i] = __uint_as_float(w[i] << 16);
        v[r + 2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      }
    }
  } else {
#pragma unroll
    for (int r = 0; r < R; r += 4) {
      float t4[4];
      load4(p + r, t4);
      v[r] = t4[0]; v[r + 1] = t4[1]; v[r + 2] = t4[2]; v[r + 3] = t4[3];
    }
  }
}

template <typename T, int R>
__global__ void __launch_bounds__(REC_THREADS)
mlstm_recurrence_async_kernel(const T* __restrict__ proj, long long ld, int q_off, int k_off, int v_off, float q_scale,
                              const float* __restrict__ keep, const float* __restrict__ take,
                              float* __restrict__ state, long long state_stride, const int* __restrict__ cu_seqlens,
                              const int* __restrict__ slots, float* __restrict__ o, float* __restrict__ nq, int heads,
                              int dim, int vdim, int L) {
  extern __shared__ __align__(16) unsigned char sm_raw[];
  const int h = blockIdx.y, seq = blockIdx.z;
  const int begin = cu_seqlens[seq], end = cu_seqlens[seq + 1];
  if (begin >= end) return;
  const int cols = REC_THREADS / L;                 // columns of this block; a block never straddles column vdim
  const int dim_pad = L * R;
  const int col0 = blockIdx.x * cols;
  const int my = threadIdx.x / L, sub = threadIdx.x % L;
  const int col = col0 + my;
  const bool live = col <= vdim;
  const bool has_v = col0 < vdim;                   // else: the block of the column of n
  // a buffer: q [AHEAD][dim_pad] T, k [AHEAD][dim_pad] T, v [AHEAD][cols] T, keep [AHEAD] float, take [AHEAD] float
  const size_t qk_bytes = (size_t)REC_AHEAD * dim_pad * sizeof(T);
  const size_t v_bytes = (size_t)REC_AHEAD * cols * sizeof(T);
  const size_t buf_bytes = 2 * qk_bytes + v_bytes + 2 * REC_AHEAD * sizeof(float);
  auto q_of = [&](int b) { return reinterpret_cast<T*>(sm_raw + b * buf_bytes); };
  auto k_of = [&](int b) { return reinterpret_cast<T*>(sm_raw + b * buf_bytes + qk_bytes); };
  auto v_of = [&](int b) { return reinterpret_cast<T*>(sm_raw + b * buf_bytes + 2 * qk_bytes); };
  auto g_of = [&](int b) { return reinterpret_cast<float*>(sm_raw + b * buf_bytes + 2 * qk_bytes + v_bytes); };
  if (dim_pad > dim) {                              // rows past dim stay zero in both buffers
    for (int b = 0; b < 2; ++b)
      for (int i = threadIdx.x; i < REC_AHEAD * (dim_pad - dim); i += REC_THREADS) {
        const int j = i / (dim_pad - dim), d = dim + i % (dim_pad - dim);
        q_of(b)[j * dim_pad + d] = hb::from_f32<T>(0.f);
        k_of(b)[j * dim_pad + d] = hb::from_f32<T>(0.f);
      }
  }
  constexpr int PER16 = 16 / (int)sizeof(T);
  const int row_runs = dim / PER16, v_runs = cols / PER16;
  auto issue = [&](int t0, int b) {
    const int count = min(REC_AHEAD, end - t0);
    for (int i = threadIdx.x; i < count * row_runs; i += REC_THREADS) {
      const int j = i / row_runs, r = i - j * row_runs;
      const T* src = proj + (size_t)(t0 + j) * ld + (size_t)h * dim + r * PER16;
      cp_async_16(q_of(b) + j * dim_pad + r * PER16, src + q_off);
      cp_async_16(k_of(b) + j * dim_pad + r * PER16, src + k_off);
    }
    if (has_v)
      for (int i = threadIdx.x; i < count * v_runs; i += REC_THREADS) {
        const int j = i / v_runs, r = i - j * v_runs;
        cp_async_16(v_of(b) + j * cols + r * PER16, proj + (size_t)(t0 + j) * ld + v_off + (size_t)h * vdim + col0 + r * PER16);
      }
    for (int i = threadIdx.x; i < 2 * count; i += REC_THREADS) {
      const int j = i >> 1;
      cp_async_4(g_of(b) + (i & 1) * REC_AHEAD + j, ((i & 1) ? take : keep) + (size_t)(t0 + j) * heads + h);
    }
    cp_async_commit();
  };
  float* S_col = state + (size_t)slots[seq] * state_stride + ((size_t)h * (vdim + 1) + (live ? col : 0)) * dim;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int d = sub * R + r;
    S[r] = (live && d < dim) ? S_col[d] : 0.f;
  }
  // lane 0 of a live column writes: a value column into o, the column of n into nq
  const bool writer = sub == 0 && live;
  float* out_ptr = col < vdim ? o + ((size_t)begin * heads + h) * vdim + col : nq + (size_t)begin * heads + h;
  const size_t out_stride = col < vdim ? (size_t)heads * vdim : (size_t)heads;
  const float fixed_v = col == vdim ? 1.f : 0.f;
  issue(begin, 0);
  int b = 0;
  for (int t0 = begin; t0 < end; t0 += REC_AHEAD, b ^= 1) {
    const int count = min(REC_AHEAD, end - t0);
    if (t0 + REC_AHEAD < end) {
      issue(t0 + REC_AHEAD, b ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const T* qp = q_of(b) + sub * R;
    const T* kp = k_of(b) + sub * R;
    const T* vp = v_of(b) + my;
    const float* gb = g_of(b);
    float* op = out_ptr + (size_t)(t0 - begin) * out_stride;      // read by writers only
#pragma unroll 2
    for (int j = 0; j < count; ++j, qp += dim_pad, kp += dim_pad, vp += cols, op += out_stride) {
      const float a = gb[j];
      const float bv = gb[REC_AHEAD + j] * (has_v ? hb::to_f32(*vp) : fixed_v);
      float q8[R], k8[R];
      load_row<R>(qp, q8);
      load_row<R>(kp, k8);
      float acc0 = 0.f, acc1 = 0.f;          // two chains: the sum over a lane's rows is not one long dependency
#pragma unroll
      for (int r = 0; r < R; r += 2) {
        S[r] = fmaf(bv, k8[r], a * S[r]);
        S[r + 1] = fmaf(bv, k8[r + 1], a * S[r + 1]);
        acc0 = fmaf(S[r], q8[r], acc0);
        acc1 = fmaf(S[r + 1], q8[r + 1], acc1);
      }
      float acc = acc0 + acc1;
      for (int off = L >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (writer) *op = acc * q_scale;
    }
    __syncthreads();              // the buffer is free for the tokens after the next ones
  }
  if (live) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int d = sub * R + r;
      if (d < dim) S_col[d] = S[r];
    }
  }
}

// One warp per (token, head): h_j = o_j / (max(|n.q|, floor) + 1e-6); y = h / sqrt(mean h^2 + eps) * w[head, j]
// * sigmoid(gate[token, head, j]); the gate is a column run of `proj`.
__global__ void mlstm_out_norm_kernel(const float* __restrict__ o, const float* __restrict__ nq,
                                      const float* __restrict__ floor_, const void* __restrict__ proj, int proj_dtype,
                                      long long ld, int g_off, const void* __restrict__ w, int w_dtype, float eps,
                                      void* __restrict__ out, int out_dtype, long long rows, int heads, int vdim) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const long long t = row / heads;
  const int h = (int)(row - t * heads);
  const float den = 1.f / (fmaxf(fabsf(nq[row]), floor_[row]) + 1e-6f);
  const float* orow = o + row * vdim;
  float ss = 0.f;
  for (int j = lane; j < vdim; j += 32) {
    const float v = orow[j] * den;
    ss += v * v;
  }
  ss = hb::warp_sum(ss);
  const float inv = rsqrtf(ss / (float)vdim + eps) * den;
  for (int j = lane; j < vdim; j += 32) {
    const float g = load_el(proj, proj_dtype, (size_t)t * ld + g_off + (size_t)h * vdim + j);
    const float y = orow[j] * inv * load_el(w, w_dtype, (size_t)h * vdim + j) / (1.f + expf(-g));
    if (out_dtype == HB_DTYPE_F32) reinterpret_cast<float*>(out)[row * vdim + j] = y;
    else reinterpret_cast<__nv_bfloat16*>(out)[row * vdim + j] = __float2bfloat16_rn(y);
  }
}

bool dtype_ok(int d) { return d == HB_DTYPE_F32 || d == HB_DTYPE_BF16; }

}  // namespace

extern "C" int hb_mlstm_gates(const float* z, const float* bias_i, const float* bias_f, float cap, float* state,
                              long long state_stride, long long m_off, const int* cu_seqlens, const int* slots,
                              float* keep, float* take, float* floor_, int n_seqs, int heads, cudaStream_t stream) {
  if (!z || !state || !cu_seqlens || !slots || !keep || !take || !floor_ || n_seqs < 0 || heads <= 0 || !(cap > 0.f))
    return HB_ERR_BAD_ARG;
  if (n_seqs == 0) return HB_OK;
  if (n_seqs > 65535) return HB_ERR_UNSUPPORTED;
  mlstm_gates_kernel<<<dim3(heads, n_seqs), GATE_THREADS, 0, stream>>>(z, bias_i, bias_f, cap, state, state_stride, m_off,
                                                                        cu_seqlens, slots, keep, take, floor_, heads);
  HB_LAUNCH_CHECK();
  return HB_OK;
}

// rows_per_lane: 0 = chosen by dim (4 up to 32, 8 up to 256, 16 up to 512, 32 up to 1024; measured at 2,048 tokens of
// 16 heads of 128: 636, 558, 656 and 867 us with 4, 8, 16 and 32 rows), or one of 4, 8, 16, 32
// (the sums over a column's rows then run in another order: results move by rounding).
extern "C" int hb_mlstm_recurrence(const void* proj, int proj_dtype, long long ld, int q_off, int k_off, int v_off,
                                   float q_scale, const float* keep, const float* take, float* state,
                                   long long state_stride, const int* cu_seqlens, const int* slots, float* o, float* nq,
                                   int n_seqs, int heads, int dim, int vdim, int rows_per_lane, cudaStream_t stream) {
  if (!proj || !keep || !take || !state || !cu_seqlens || !slots || !o || !nq || n_seqs < 0 || heads <= 0 || dim <= 0 ||
      vdim <= 0 || !dtype_ok(proj_dtype))
    return HB_ERR_BAD_ARG;
  if (n_seqs == 0) return HB_OK;
  if (dim > 1024 || n_seqs > 65535 || heads > 65535) return HB_ERR_UNSUPPORTED;
  int R = rows_per_lane;
  if (R == 0) R = dim <= 32 ? 4 : (dim <= 256 ? 8 : (dim <= 512 ? 16 : 32));
  if (!(R == 4 || R == 8 || R == 16 || R == 32) || 32 * R < dim) return HB_ERR_BAD_ARG;
  int L = 1;
  while (L * R < dim) L *= 2;
  const int cols_per_block = REC_THREADS / L;
  const dim3 grid((vdim + 1 + cols_per_block - 1) / cols_per_block, heads, n_seqs);
  {
    // rows and column runs of whole 16-byte pieces, and no block that holds both values and the column of n:
    // the kernel that stages the next tokens with cp.async
    const int el = proj_dtype == HB_DTYPE_F32 ? 4 : 2, per16 = 16 / el;
    const bool aligned = dim % per16 == 0 && vdim % cols_per_block == 0 && cols_per_block % per16 == 0 && ld % per16 == 0 &&
                         q_off % per16 == 0 && k_off % per16 == 0 && v_off % per16 == 0 &&
                         (reinterpret_cast<uintptr_t>(proj) & 15) == 0;
    const size_t asmem = 2 * ((size_t)REC_AHEAD * (2 * L * R + cols_per_block) * el + 2 * REC_AHEAD * sizeof(float));
    if (aligned && asmem <= 200 * 1024) {
#define HB_MLSTM_ASYNC(T, RR)                                                                                       \
  do {                                                                                                              \
    if (asmem > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(mlstm_recurrence_async_kernel<T, RR>,                                    \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)asmem);                \
      if (e != cudaSuccess) return (int)e;                                                                          \
    }                                                                                                               \
    mlstm_recurrence_async_kernel<T, RR><<<grid, REC_THREADS, asmem, stream>>>(                                     \
        (const T*)proj, ld, q_off, k_off, v_off, q_scale, keep, take, state, state_stride, cu_seqlens, slots, o, nq, \
        heads, dim, vdim, L);                                                                                       \
  } while (0)
#define HB_MLSTM_ASYNC_R(T)                                                                                         \
  do {                                                                                                              \
    if (R == 4) HB_MLSTM_ASYNC(T, 4);                                                                               \
    else if (R == 8) HB_MLSTM_ASYNC(T, 8);                                                                          \
    else if (R == 16) HB_MLSTM_ASYNC(T, 16);                                                                        \
    else HB_MLSTM_ASYNC(T, 32);                                                                                     \
  } while (0)
      if (proj_dtype == HB_DTYPE_F32) HB_MLSTM_ASYNC_R(float);
      else HB_MLSTM_ASYNC_R(__nv_bfloat16);
#undef HB_MLSTM_ASYNC_R
#undef HB_MLSTM_ASYNC
      HB_LAUNCH_CHECK();
      return HB_OK;
    }
  }
  const size_t smem = (size_t)REC_TOKENS * (2 * L * R + cols_per_block + 2) * sizeof(float);
#define HB_MLSTM_REC(RR)                                                                                          \
  do {                                                                                                            \
    if (smem > 48 * 1024) {                                                                                       \
      cudaError_t e = cudaFuncSetAttribute(mlstm_recurrence_kernel<RR>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem);                                                            \
      if (e != cudaSuccess) return (int)e;                                                                        \
    }                                                                                                             \
    mlstm_recurrence_kernel<RR><<<grid, REC_THREADS, smem, stream>>>(proj, proj_dtype, ld, q_off, k_off, v_off,    \
                                                                     q_scale, keep, take, state, state_stride,    \
                                                                     cu_seqlens, slots, o, nq, heads, dim, vdim, L); \
  } while (0)
  if (R == 4) HB_MLSTM_REC(4);
  else if (R == 8) HB_MLSTM_REC(8);
  else if (R == 16) HB_MLSTM_REC(16);
  else HB_MLSTM_REC(32);
#undef HB_MLSTM_REC
  HB_LAUNCH_CHECK();
  return HB_OK;
}

extern "C" int hb_mlstm_out_norm(const float* o, const float* nq, const float* floor_, const void* proj, int proj_dtype,
                                 long long ld, int g_off, const void* w, int w_dtype, float eps, void* out,
                                 int out_dtype, long long n_tokens, int heads, int vdim, cudaStream_t stream) {
  if (!o || !nq || !floor_ || !proj || !w || !out || n_tokens < 0 || heads <= 0 || vdim <= 0 || !dtype_ok(proj_dtype) ||
      !dtype_ok(w_dtype) || !dtype_ok(out_dtype))
    return HB_ERR_BAD_ARG;
  const long long rows = n_tokens * heads;
  if (rows == 0) return HB_OK;
  const int warps = 8;
  const long long blocks = (rows + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return HB_ERR_UNSUPPORTED;
  mlstm_out_norm_kernel<<<(int)blocks, warps * 32, 0, stream>>>(o, nq, floor_, proj, proj_dtype, ld, g_off, w, w_dtype, eps,
                                                               out, out_dtype, rows, heads, vdim);
  HB_LAUNCH_CHECK();
  return HB_OK;
}
