// K8-class row kernels for the operations either side of the FFN / MoE /
// attention path in a transformer block: layer / RMS normalisation, embedding
// row gather, and softmax cross-entropy over a (possibly mesh-split) vocabulary.
// All are HBM-bound: every input element is read once and every output element
// written once, 16 bytes per thread per access where the row length allows.
//
// They replace, per slice, the op chains of
//   layer_norm        mesh_tensorflow/layers.py:950-979
//   rms norm          mesh_tensorflow/transformer/transformer.py:493-516
//   gather/embedding  mesh_tensorflow/ops.py:5231-5251, layers.py:2049-2073
//                     (a one-hot einsum in the reference)
//   softmax_cross_entropy_with_logits   layers.py:1062-1117, with
//                     reduce_logsumexp ops.py:5493-5520
// Arithmetic is fp32 whatever the storage type, with one rounding at the store.

#include "common.cuh"

namespace mtfc {
namespace {

constexpr int kRowWarps = 8;           // warps (rows in flight) per CTA
constexpr int kMaxVecPerLane = 8;      // 16-byte vectors a lane keeps in registers

template <typename T> struct VecTraits;
template <> struct VecTraits<float> { static constexpr int N = 4; };
template <> struct VecTraits<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float (&f)[VecTraits<T>::N]);
template <>
__device__ __forceinline__ void load_vec<float>(const float* p, float (&f)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <>
__device__ __forceinline__ void load_vec<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
template <typename T>
__device__ __forceinline__ void store_vec(T* p, const float (&f)[VecTraits<T>::N]);
template <>
__device__ __forceinline__ void store_vec<float>(float* p, const float (&f)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <>
__device__ __forceinline__ void store_vec<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
  return v;
}

// One warp per row, the row held in registers (cols <= 32 * kMaxVecPerLane * N).
//   centered: y = (x - mean) * rsqrt(mean((x - mean)^2) + eps) * scale + bias
//   else    : y = x * rsqrt(mean(x^2) + eps) * scale
// scale / bias may be null (1 / 0).
template <typename T>
__global__ void __launch_bounds__(32 * kRowWarps)
norm_rows_kernel(const T* __restrict__ x, const T* __restrict__ scale, const T* __restrict__ bias,
                 T* __restrict__ y, long long rows, int cols, float eps, int centered) {
  constexpr int N = VecTraits<T>::N;
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kRowWarps;
  const int nvec = cols / N;
  const float inv = 1.0f / (float)cols;
  for (long long r = warp; r < rows; r += nwarps) {
    const T* src = x + r * cols;
    float v[kMaxVecPerLane][N];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxVecPerLane; ++j) {
      const int i = lane + 32 * j;
      if (i < nvec) {
        load_vec<T>(src + (long long)i * N, v[j]);
#pragma unroll
        for (int e = 0; e < N; ++e) sum += centered ? v[j][e] : v[j][e] * v[j][e];
      }
    }
    sum = warp_sum(sum);
    float mean = 0.f, var;
    if (centered) {
      mean = sum * inv;
      float sq = 0.f;
#pragma unroll
      for (int j = 0; j < kMaxVecPerLane; ++j) {
        if (lane + 32 * j < nvec) {
#pragma unroll
          for (int e = 0; e < N; ++e) {
            const float d = v[j][e] - mean;
            sq += d * d;
          }
        }
      }
      var = warp_sum(sq) * inv;
    } else {
      var = sum * inv;
    }
    const float rstd = rsqrtf(var + eps);
    T* dst = y + r * cols;
#pragma unroll
    for (int j = 0; j < kMaxVecPerLane; ++j) {
      const int i = lane + 32 * j;
      if (i < nvec) {
        float s[N], b[N];
        if (scale) load_vec<T>(scale + (long long)i * N, s);
        if (bias) load_vec<T>(bias + (long long)i * N, b);
#pragma unroll
        for (int e = 0; e < N; ++e) {
          float o = (v[j][e] - mean) * rstd;
          if (scale) o *= s[e];
          if (bias) o += b[e];
          v[j][e] = o;
        }
        store_vec<T>(dst + (long long)i * N, v[j]);
      }
    }
  }
}

// Any row length: one warp per row, the row read up to three times (the repeats
// come from L1/L2), element by element.
template <typename T>
__global__ void __launch_bounds__(32 * kRowWarps)
norm_rows_general_kernel(const T* __restrict__ x, const T* __restrict__ scale,
                         const T* __restrict__ bias, T* __restrict__ y, long long rows, int cols,
                         float eps, int centered) {
  const int lane = threadIdx.x & 31;
  const long long warp = (long long)blockIdx.x * kRowWarps + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * kRowWarps;
  const float inv = 1.0f / (float)cols;
  for (long long r = warp; r < rows; r += nwarps) {
    const T* src = x + r * cols;
    float sum = 0.f;
    for (int i = lane; i < cols; i += 32) {
      const float f = to_f32<T>(src[i]);
      sum += centered ? f : f * f;
    }
    sum = warp_sum(sum);
    float mean = 0.f, var;
    if (centered) {
      mean = sum * inv;
      float sq = 0.f;
      for (int i = lane; i < cols; i += 32) {
        const float d = to_f32<T>(src[i]) - mean;
        sq += d * d;
      }
      var = warp_sum(sq) * inv;
    } else {
      var = sum * inv;
    }
    const float rstd = rsqrtf(var + eps);
    T* dst = y + r * cols;
    for (int i = lane; i < cols; i += 32) {
      float o = (to_f32<T>(src[i]) - mean) * rstd;
      if (scale) o *= to_f32<T>(scale[i]);
      if (bias) o += to_f32<T>(bias[i]);
      dst[i] = from_f32<T>(o);
    }
  }
}

// out[r, :] = table[idx[r] - first_row, :] when that row is held here, else zeros.
// One warp per output row, 16-byte vectors.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ table, const int* __restrict__ idx,
                   uint4* __restrict__ out, long long rows, long long table_rows, int first_row,
                   int vec_per_row) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = warp; r < rows; r += nwarps) {
    const long long src_row = (long long)idx[r] - first_row;
    uint4* dst = out + r * vec_per_row;
    if (src_row >= 0 && src_row < table_rows) {
      const uint4* src = table + src_row * vec_per_row;
      for (int v = lane; v < vec_per_row; v += 32) dst[v] = src[v];
    } else {
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int v = lane; v < vec_per_row; v += 32) dst[v] = z;
    }
  }
}

// Cross-entropy statistics of one slice of the vocabulary, one CTA per row:
//   row_max[r] = max_v x[r, v]
//   row_sum[r] = sum_v exp(x[r, v] - row_max[r])
//   picked[r]  = x[r, target[r] - first_col] if the target column is held here, else 0
// Slices combine as max over slices of row_max, then sum of row_sum * exp(row_max - max).
template <typename T>
__global__ void __launch_bounds__(256)
xent_stats_kernel(const T* __restrict__ x, const int* __restrict__ target, long long rows, int cols,
                  int first_col, float* __restrict__ row_max, float* __restrict__ row_sum,
                  float* __restrict__ picked) {
  constexpr int N = VecTraits<T>::N;
  __shared__ float sm_m[8], sm_s[8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool vec_ok = cols % N == 0;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* src = x + r * cols;
    float m = -INFINITY, s = 0.f;   // running max and sum of exp(x - m)
    if (vec_ok) {
      const int nvec = cols / N;
      for (int i = tid; i < nvec; i += blockDim.x) {
        float f[N];
        load_vec<T>(src + (long long)i * N, f);
        float vm = f[0];
#pragma unroll
        for (int e = 1; e < N; ++e) vm = fmaxf(vm, f[e]);
        if (vm > m) {
          s *= __expf(m - vm);   // m = -inf the first time: s is 0 and stays 0
          m = vm;
        }
#pragma unroll
        for (int e = 0; e < N; ++e) s += __expf(f[e] - m);
      }
    } else {
      for (int i = tid; i < cols; i += blockDim.x) {
        const float f = to_f32<T>(src[i]);
        if (f > m) {
          s *= __expf(m - f);
          m = f;
        }
        s += __expf(f - m);
      }
    }
    // combine (m, s) pairs: warp, then CTA
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, sft);
      const float os = __shfl_xor_sync(0xffffffffu, s, sft);
      const float nm = fmaxf(m, om);
      s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
      m = nm;
    }
    if (lane == 0) { sm_m[warp] = m; sm_s[warp] = s; }
    __syncthreads();
    if (tid == 0) {
      float gm = sm_m[0], gs = sm_s[0];
      for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
        const float nm = fmaxf(gm, sm_m[w]);
        gs = (gm == -INFINITY ? 0.f : gs * __expf(gm - nm)) +
             (sm_m[w] == -INFINITY ? 0.f : sm_s[w] * __expf(sm_m[w] - nm));
        gm = nm;
      }
      row_max[r] = gm;
      row_sum[r] = gs;
      const long long c = (long long)target[r] - first_col;
      picked[r] = (c >= 0 && c < cols) ? to_f32<T>(src[c]) : 0.f;
    }
    __syncthreads();
  }
}

// dlogits[r, v] = dloss[r] * (coef[r] * exp(x[r, v] - log_z[r]) - [v + first_col == target[r]])
// (coef = 1 + 2 * z_loss * log_z carries the z-loss term).
template <typename T>
__global__ void __launch_bounds__(256)
xent_grad_kernel(const T* __restrict__ x, const int* __restrict__ target,
                 const float* __restrict__ log_z, const float* __restrict__ dloss, float z_loss,
                 long long rows, int cols, int first_col, T* __restrict__ dx) {
  constexpr int N = VecTraits<T>::N;
  const bool vec_ok = cols % N == 0;
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const T* src = x + r * cols;
    T* dst = dx + r * cols;
    const float lz = log_z[r], g = dloss[r];
    const float coef = 1.0f + 2.0f * z_loss * lz;
    const long long hot = (long long)target[r] - first_col;
    if (vec_ok) {
      const int nvec = cols / N;
      for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        float f[N];
        load_vec<T>(src + (long long)i * N, f);
#pragma unroll
        for (int e = 0; e < N; ++e) {
          const float p = coef * __expf(f[e] - lz);
          f[e] = g * (p - (((long long)i * N + e) == hot ? 1.0f : 0.0f));
        }
        store_vec<T>(dst + (long long)i * N, f);
      }
    } else {
      for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float p = coef * __expf(to_f32<T>(src[i]) - lz);
        dst[i] = from_f32<T>(g * (p - (i == hot ? 1.0f : 0.0f)));
      }
    }
  }
}

// Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3"):
// counter (c0..c3), key (k0, k1) -> four 32-bit words.
__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
    c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

// Element i takes word i % 4 of block i / 4 of the stream keyed by `seed`.
// uniform: a + (b - a) * u, u = (word >> 8) * 2^-24 in [0, 1).
// normal : a + b * z, z from Box-Muller on the block's word pairs (0,1) / (2,3):
//          r = sqrt(-2 log(1 - u0)), z = r cos(2 pi u1) for even i, r sin(2 pi u1) for odd i.
template <typename T>
__global__ void random_kernel(T* __restrict__ out, long long n, uint32_t seed_lo, uint32_t seed_hi,
                              int normal, float a, float b) {
  const long long step = (long long)gridDim.x * blockDim.x;
  const long long blocks = (n + 3) / 4;
  for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < blocks; q += step) {
    uint32_t c[4] = {(uint32_t)q, (uint32_t)((unsigned long long)q >> 32), 0u, 0u};
    philox4x32_10(c, seed_lo, seed_hi);
    float v[4];
    if (normal) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float u0 = (float)(c[2 * h] >> 8) * (1.0f / 16777216.0f);
        const float u1 = (float)(c[2 * h + 1] >> 8) * (1.0f / 16777216.0f);
        const float r = sqrtf(-2.0f * logf(1.0f - u0));
        float sn, cs;
        sincosf(6.283185307179586f * u1, &sn, &cs);
        v[2 * h] = __fadd_rn(a, __fmul_rn(b, __fmul_rn(r, cs)));
        v[2 * h + 1] = __fadd_rn(a, __fmul_rn(b, __fmul_rn(r, sn)));
      }
    } else {
#pragma unroll
      // separately rounded multiply and add (no fused multiply-add), so that the
      // values can be restated exactly with ordinary float32 arithmetic
      for (int e = 0; e < 4; ++e)
        v[e] = __fadd_rn(a, __fmul_rn(__fsub_rn(b, a), (float)(c[e] >> 8) * (1.0f / 16777216.0f)));
    }
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (4 * q + e < n) out[4 * q + e] = from_f32<T>(v[e]);
  }
}

bool aligned16p(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace mtfc

using namespace mtfc;

extern "C" {

int mtfc_norm_rows(const void* x, const void* scale, const void* bias, void* y, int dtype,
                   int64_t rows, int64_t cols, float epsilon, int32_t centered, void* stream) {
  if (rows < 0 || cols < 1 || cols > INT32_MAX) return fail(MTFC_ERR_SHAPE, "norm_rows: bad extents");
  if (rows == 0) return MTFC_OK;
  if (!x || !y) return fail(MTFC_ERR_SHAPE, "norm_rows: null argument");
  if (dtype != MTFC_F32 && dtype != MTFC_BF16)
    return fail(MTFC_ERR_UNSUPPORTED, "norm_rows: dtype %d", dtype);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int n = dtype == MTFC_F32 ? 4 : 8;
  const bool fast = cols % n == 0 && cols / n <= 32 * kMaxVecPerLane && aligned16p(x) && aligned16p(y) &&
                    (!scale || aligned16p(scale)) && (!bias || aligned16p(bias));
  const unsigned grid = grid_for(rows, kRowWarps, 8);
  if (dtype == MTFC_F32) {
    auto px = static_cast<const float*>(x);
    auto ps = static_cast<const float*>(scale);
    auto pb = static_cast<const float*>(bias);
    auto py = static_cast<float*>(y);
    if (fast)
      norm_rows_kernel<float><<<grid, 32 * kRowWarps, 0, s>>>(px, ps, pb, py, rows, (int)cols, epsilon, centered);
    else
      norm_rows_general_kernel<float><<<grid, 32 * kRowWarps, 0, s>>>(px, ps, pb, py, rows, (int)cols, epsilon, centered);
  } else {
    auto px = static_cast<const __nv_bfloat16*>(x);
    auto ps = static_cast<const __nv_bfloat16*>(scale);
    auto pb = static_cast<const __nv_bfloat16*>(bias);
    auto py = static_cast<__nv_bfloat16*>(y);
    if (fast)
      norm_rows_kernel<__nv_bfloat16><<<grid, 32 * kRowWarps, 0, s>>>(px, ps, pb, py, rows, (int)cols, epsilon, centered);
    else
      norm_rows_general_kernel<__nv_bfloat16><<<grid, 32 * kRowWarps, 0, s>>>(px, ps, pb, py, rows, (int)cols, epsilon, centered);
  }
  MTFC_LAUNCH_CHECK("norm_rows_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_random(void* out, int dtype, int64_t n, int32_t normal, uint64_t seed, float a, float b,
                void* stream) {
  if (n < 0) return fail(MTFC_ERR_SHAPE, "random: negative size");
  if (n == 0) return MTFC_OK;
  if (!out) return fail(MTFC_ERR_SHAPE, "random: null argument");
  if (dtype != MTFC_F32 && dtype != MTFC_BF16)
    return fail(MTFC_ERR_UNSUPPORTED, "random: dtype %d", dtype);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint32_t lo = (uint32_t)seed, hi = (uint32_t)(seed >> 32);
  const unsigned grid = grid_for((n + 3) / 4, 256);
  if (dtype == MTFC_F32)
    random_kernel<float><<<grid, 256, 0, s>>>(static_cast<float*>(out), n, lo, hi, normal, a, b);
  else
    random_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(out), n, lo, hi,
                                                      normal, a, b);
  MTFC_LAUNCH_CHECK("random_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_gather_rows(const void* table, const int32_t* indices, void* out, int64_t rows,
                     int64_t table_rows, int32_t first_row, int64_t row_bytes, void* stream) {
  if (rows < 0 || table_rows < 0) return fail(MTFC_ERR_SHAPE, "gather_rows: bad extents");
  if (rows == 0) return MTFC_OK;
  if (!table || !indices || !out) return fail(MTFC_ERR_SHAPE, "gather_rows: null argument");
  if (row_bytes < 16 || row_bytes % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "gather_rows: row of %lld bytes is not a multiple of 16", (long long)row_bytes);
  if (!aligned16p(table) || !aligned16p(out))
    return fail(MTFC_ERR_SHAPE, "gather_rows: buffers must be 16-byte aligned");
  gather_rows_kernel<<<grid_for(rows * 32, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(table), indices, static_cast<uint4*>(out), rows, table_rows,
      first_row, (int)(row_bytes / 16));
  MTFC_LAUNCH_CHECK("gather_rows_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_xent_stats(const void* logits, int dtype, const int32_t* targets, int64_t rows, int64_t cols,
                    int32_t first_col, float* row_max, float* row_sum, float* picked, void* stream) {
  if (rows < 0 || cols < 1 || cols > INT32_MAX) return fail(MTFC_ERR_SHAPE, "xent_stats: bad extents");
  if (rows == 0) return MTFC_OK;
  if (!logits || !targets || !row_max || !row_sum || !picked)
    return fail(MTFC_ERR_SHAPE, "xent_stats: null argument");
  if (dtype != MTFC_F32 && dtype != MTFC_BF16)
    return fail(MTFC_ERR_UNSUPPORTED, "xent_stats: dtype %d", dtype);
  // rows whose length is a multiple of the vector width are read 16 bytes at a time
  if ((cols % (dtype == MTFC_F32 ? 4 : 8)) == 0 && !aligned16p(logits))
    return fail(MTFC_ERR_SHAPE, "xent_stats: logits must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = grid_for(rows, 1, 8);
  if (dtype == MTFC_F32)
    xent_stats_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(logits), targets, rows,
                                                  (int)cols, first_col, row_max, row_sum, picked);
  else
    xent_stats_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(logits), targets, rows, (int)cols, first_col, row_max,
        row_sum, picked);
  MTFC_LAUNCH_CHECK("xent_stats_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_xent_grad(const void* logits, int dtype, const int32_t* targets, const float* log_z,
                   const float* dloss, float z_loss, int64_t rows, int64_t cols, int32_t first_col,
                   void* dlogits, void* stream) {
  if (rows < 0 || cols < 1 || cols > INT32_MAX) return fail(MTFC_ERR_SHAPE, "xent_grad: bad extents");
  if (rows == 0) return MTFC_OK;
  if (!logits || !targets || !log_z || !dloss || !dlogits)
    return fail(MTFC_ERR_SHAPE, "xent_grad: null argument");
  if (dtype != MTFC_F32 && dtype != MTFC_BF16)
    return fail(MTFC_ERR_UNSUPPORTED, "xent_grad: dtype %d", dtype);
  if ((cols % (dtype == MTFC_F32 ? 4 : 8)) == 0 && (!aligned16p(logits) || !aligned16p(dlogits)))
    return fail(MTFC_ERR_SHAPE, "xent_grad: buffers must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = grid_for(rows, 1, 8);
  if (dtype == MTFC_F32)
    xent_grad_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float*>(logits), targets, log_z,
                                                 dloss, z_loss, rows, (int)cols, first_col,
                                                 static_cast<float*>(dlogits));
  else
    xent_grad_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(logits), targets, log_z, dloss, z_loss, rows, (int)cols,
        first_col, static_cast<__nv_bfloat16*>(dlogits));
  MTFC_LAUNCH_CHECK("xent_grad_kernel");
  count_launch(1);
  return MTFC_OK;
}

}  // extern "C"
