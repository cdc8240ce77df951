// K7 / K8: the slice-local array operations an op-by-op lowering needs —
// casts and unary maps, binary maps with broadcasting, strided copies
// (transpose / slice / concat / pack / unpack), multiply-and-reduce over
// arbitrary axes, arg-max / top-k / gather along the last axis, one-hot,
// fill and range.  They replace the tf.* calls made inside
// MeshImpl.slicewise closures (mesh_tensorflow/ops.py:1710-1723, 2066-2084,
// 2320-2338, 3843-3851, 4937-4958) and the tf.split / tf.concat / tf.slice
// calls around the collectives (placement_mesh_impl.py:436-440, 487, 509-510).
//
// All are HBM-bound grid-stride kernels; grids are sized in whole multiples
// of the SM count.  float32 / bfloat16 / int32 storage; floating arithmetic
// is done in float32 and rounded once at the store; bool is int32 0/1.

#include "common.cuh"

namespace mtfc {
namespace {

constexpr int kThreads = 256;

struct Dims {
  int ndim;
  long long shape[MTFC_MAX_DIMS];
  long long stride[4][MTFC_MAX_DIMS];
};

template <typename T> struct Compute { using type = float; };
template <> struct Compute<int> { using type = int; };

template <typename T> __device__ __forceinline__ typename Compute<T>::type ld(const T* p, long long i);
template <> __device__ __forceinline__ float ld<float>(const float* p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}
template <> __device__ __forceinline__ int ld<int>(const int* p, long long i) { return p[i]; }

template <typename T, typename C> __device__ __forceinline__ void st(T* p, long long i, C v);
template <> __device__ __forceinline__ void st<float, float>(float* p, long long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void st<__nv_bfloat16, float>(__nv_bfloat16* p, long long i, float v) {
  p[i] = __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ void st<int, float>(int* p, long long i, float v) {
  p[i] = (int)truncf(v);
}
template <> __device__ __forceinline__ void st<float, int>(float* p, long long i, int v) { p[i] = (float)v; }
template <> __device__ __forceinline__ void st<__nv_bfloat16, int>(__nv_bfloat16* p, long long i, int v) {
  p[i] = __float2bfloat16_rn((float)v);
}
template <> __device__ __forceinline__ void st<int, int>(int* p, long long i, int v) { p[i] = v; }

// ------------------------------------------------------------------- unary
__device__ __forceinline__ float unary_f(int op, float x) {
  switch (op) {
    case MTFC_UNARY_IDENTITY: return x;
    case MTFC_UNARY_RELU: return x > 0.f ? x : 0.f;
    case MTFC_UNARY_EXP: return expf(x);
    case MTFC_UNARY_LOG: return logf(x);
    case MTFC_UNARY_NEGATIVE: return -x;
    case MTFC_UNARY_RECIPROCAL: return 1.0f / x;
    case MTFC_UNARY_SQRT: return sqrtf(x);
    case MTFC_UNARY_RSQRT: return 1.0f / sqrtf(x);
    case MTFC_UNARY_SQUARE: return x * x;
    case MTFC_UNARY_TANH: return tanhf(x);
    case MTFC_UNARY_SIGMOID: return 1.0f / (1.0f + expf(-x));
    case MTFC_UNARY_SIGN: return (float)((x > 0.f) - (x < 0.f));
    case MTFC_UNARY_LOGICAL_NOT: return x != 0.f ? 0.f : 1.f;
    case MTFC_UNARY_NONZERO: return x != 0.f ? 1.f : 0.f;
    default: return x;
  }
}
__device__ __forceinline__ int unary_i(int op, int x) {
  switch (op) {
    case MTFC_UNARY_RELU: return x > 0 ? x : 0;
    case MTFC_UNARY_NEGATIVE: return -x;
    case MTFC_UNARY_SQUARE: return x * x;
    case MTFC_UNARY_SIGN: return (x > 0) - (x < 0);
    case MTFC_UNARY_LOGICAL_NOT: return x != 0 ? 0 : 1;
    case MTFC_UNARY_NONZERO: return x != 0 ? 1 : 0;
    default: return x;
  }
}
__device__ __forceinline__ float apply_unary(int op, float x) { return unary_f(op, x); }
__device__ __forceinline__ int apply_unary(int op, int x) { return unary_i(op, x); }

template <typename TI, typename TO>
__global__ void unary_kernel(int op, const TI* __restrict__ x, TO* __restrict__ y, long long n) {
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
    st<TO>(y, i, apply_unary(op, ld<TI>(x, i)));
}

// ------------------------------------------------------------------ binary
__device__ __forceinline__ float binary_f(int op, float a, float b) {
  switch (op) {
    case MTFC_BINARY_ADD: return a + b;
    case MTFC_BINARY_SUB: return a - b;
    case MTFC_BINARY_MULTIPLY: return a * b;
    case MTFC_BINARY_DIVIDE: return a / b;
    case MTFC_BINARY_MAXIMUM: return fmaxf(a, b);
    case MTFC_BINARY_MINIMUM: return fminf(a, b);
    case MTFC_BINARY_FLOORDIV: return floorf(a / b);
    case MTFC_BINARY_MOD: { float r = fmodf(a, b); return (r != 0.f && ((r < 0.f) != (b < 0.f))) ? r + b : r; }
    case MTFC_BINARY_LESS: return a < b;
    case MTFC_BINARY_GREATER: return a > b;
    case MTFC_BINARY_LESS_EQUAL: return a <= b;
    case MTFC_BINARY_GREATER_EQUAL: return a >= b;
    case MTFC_BINARY_EQUAL: return a == b;
    case MTFC_BINARY_NOT_EQUAL: return a != b;
    case MTFC_BINARY_LOGICAL_AND: return (a != 0.f) && (b != 0.f);
    case MTFC_BINARY_LOGICAL_OR: return (a != 0.f) || (b != 0.f);
    case MTFC_BINARY_SELECT_POSITIVE: return b > 0.f ? a : 0.f;
    default: return 0.f;
  }
}
__device__ __forceinline__ int floordiv_i(int a, int b) {
  int q = a / b;
  return ((a % b != 0) && ((a < 0) != (b < 0))) ? q - 1 : q;
}
__device__ __forceinline__ int binary_i(int op, int a, int b) {
  switch (op) {
    case MTFC_BINARY_ADD: return a + b;
    case MTFC_BINARY_SUB: return a - b;
    case MTFC_BINARY_MULTIPLY: return a * b;
    case MTFC_BINARY_DIVIDE: return b != 0 ? a / b : 0;
    case MTFC_BINARY_MAXIMUM: return a > b ? a : b;
    case MTFC_BINARY_MINIMUM: return a < b ? a : b;
    case MTFC_BINARY_FLOORDIV: return b != 0 ? floordiv_i(a, b) : 0;
    case MTFC_BINARY_MOD: return b != 0 ? a - floordiv_i(a, b) * b : 0;
    case MTFC_BINARY_LESS: return a < b;
    case MTFC_BINARY_GREATER: return a > b;
    case MTFC_BINARY_LESS_EQUAL: return a <= b;
    case MTFC_BINARY_GREATER_EQUAL: return a >= b;
    case MTFC_BINARY_EQUAL: return a == b;
    case MTFC_BINARY_NOT_EQUAL: return a != b;
    case MTFC_BINARY_LOGICAL_AND: return (a != 0) && (b != 0);
    case MTFC_BINARY_LOGICAL_OR: return (a != 0) || (b != 0);
    case MTFC_BINARY_SELECT_POSITIVE: return b > 0 ? a : 0;
    default: return 0;
  }
}
__device__ __forceinline__ float apply_binary(int op, float a, float b) { return binary_f(op, a, b); }
__device__ __forceinline__ int apply_binary(int op, int a, int b) { return binary_i(op, a, b); }

// out is contiguous over dims.shape; input k is addressed with dims.stride[k].
template <typename TI, typename TO>
__global__ void binary_kernel(int op, const TI* __restrict__ a, const TI* __restrict__ b,
                              double scalar_b, TO* __restrict__ out, Dims dims, long long n) {
  using C = typename Compute<TI>::type;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    long long rem = i, oa = 0, ob = 0;
#pragma unroll 1
    for (int d = dims.ndim - 1; d >= 0; --d) {
      const long long c = rem % dims.shape[d];
      rem /= dims.shape[d];
      oa += c * dims.stride[0][d];
      ob += c * dims.stride[1][d];
    }
    const C va = ld<TI>(a, oa);
    const C vb = b ? ld<TI>(b, ob) : (C)scalar_b;
    st<TO>(out, i, apply_binary(op, va, vb));
  }
}

// Same-shape contiguous fast path.
template <typename TI, typename TO>
__global__ void binary_flat_kernel(int op, const TI* __restrict__ a, const TI* __restrict__ b,
                                   double scalar_b, TO* __restrict__ out, long long n) {
  using C = typename Compute<TI>::type;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    const C va = ld<TI>(a, i);
    const C vb = b ? ld<TI>(b, i) : (C)scalar_b;
    st<TO>(out, i, apply_binary(op, va, vb));
  }
}

// The same with 16-byte accesses (same dtype in and out, 16-byte aligned
// pointers): these kernels are bound by HBM, and 2- or 4-byte accesses per
// thread leave more than half of its bandwidth unused.
template <typename T>
__global__ void binary_flat_vec_kernel(int op, const T* __restrict__ a, const T* __restrict__ b,
                                       double scalar_b, T* __restrict__ out, long long nvec) {
  using C = typename Compute<T>::type;
  constexpr int V = 16 / (int)sizeof(T);
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += step) {
    const uint4 ra = reinterpret_cast<const uint4*>(a)[i];
    const uint4 rb = b ? reinterpret_cast<const uint4*>(b)[i] : make_uint4(0u, 0u, 0u, 0u);
    uint4 ro;
    const T* pa = reinterpret_cast<const T*>(&ra);
    const T* pb = reinterpret_cast<const T*>(&rb);
    T* po = reinterpret_cast<T*>(&ro);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const C va = ld<T>(pa, e);
      const C vb = b ? ld<T>(pb, e) : (C)scalar_b;
      st<T>(po, e, apply_binary(op, va, vb));
    }
    reinterpret_cast<uint4*>(out)[i] = ro;
  }
}

template <typename T>
__global__ void unary_vec_kernel(int op, const T* __restrict__ x, T* __restrict__ y, long long nvec) {
  constexpr int V = 16 / (int)sizeof(T);
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += step) {
    const uint4 rx = reinterpret_cast<const uint4*>(x)[i];
    uint4 ro;
    const T* px = reinterpret_cast<const T*>(&rx);
    T* po = reinterpret_cast<T*>(&ro);
#pragma unroll
    for (int e = 0; e < V; ++e) st<T>(po, e, apply_unary(op, ld<T>(px, e)));
    reinterpret_cast<uint4*>(y)[i] = ro;
  }
}

template <typename T>
void launch_unary_vec(int op, const void* x, void* y, long long n, cudaStream_t s) {
  constexpr int V = 16 / (int)sizeof(T);
  const long long nvec = n / V, done = nvec * V;
  unary_vec_kernel<T><<<grid_for(nvec, kThreads * 2), kThreads, 0, s>>>(
      op, static_cast<const T*>(x), static_cast<T*>(y), nvec);
  if (done < n)
    unary_kernel<T, T><<<1, kThreads, 0, s>>>(op, static_cast<const T*>(x) + done,
                                              static_cast<T*>(y) + done, n - done);
}

template <typename T>
void launch_binary_vec(int op, const void* a, const void* b, double scalar_b, void* out,
                       long long n, cudaStream_t s) {
  constexpr int V = 16 / (int)sizeof(T);
  const long long nvec = n / V, done = nvec * V;
  binary_flat_vec_kernel<T><<<grid_for(nvec, kThreads * 2), kThreads, 0, s>>>(
      op, static_cast<const T*>(a), static_cast<const T*>(b), scalar_b, static_cast<T*>(out), nvec);
  if (done < n)
    binary_flat_kernel<T, T><<<1, kThreads, 0, s>>>(
        op, static_cast<const T*>(a) + done, b ? static_cast<const T*>(b) + done : nullptr,
        scalar_b, static_cast<T*>(out) + done, n - done);
}

inline bool aligned16_all(const void* a, const void* b, const void* c) {
  return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
           reinterpret_cast<uintptr_t>(c)) & 15) == 0;
}

// ------------------------------------------------------------- strided copy
template <typename T>
__global__ void copy_strided_kernel(const T* __restrict__ src, T* __restrict__ dst, Dims dims,
                                    long long n) {
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    long long rem = i, os = 0, od = 0;
#pragma unroll 1
    for (int d = dims.ndim - 1; d >= 0; --d) {
      const long long c = rem % dims.shape[d];
      rem /= dims.shape[d];
      os += c * dims.stride[0][d];
      od += c * dims.stride[1][d];
    }
    dst[od] = src[os];
  }
}

// Rows of `row_elems` contiguous 16-byte vectors on both sides.
__global__ void copy_rows16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                   Dims dims, long long vec_per_row, long long n_vec) {
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += step) {
    const long long v = i % vec_per_row;
    long long rem = i / vec_per_row, os = 0, od = 0;
#pragma unroll 1
    for (int d = dims.ndim - 1; d >= 0; --d) {
      const long long c = rem % dims.shape[d];
      rem /= dims.shape[d];
      os += c * dims.stride[0][d];
      od += c * dims.stride[1][d];
    }
    dst[od + v] = src[os + v];
  }
}

// --------------------------------------------------- multiply-and-reduce
// out[o] = reduce_r prod_k in_k[o, r]; `out_dims` index the kept axes,
// `red_dims` the reduced ones.  One thread per output (kWarp = false) or one
// warp per output with lanes striding the reduced index (kWarp = true).
template <typename C> __device__ __forceinline__ C red_identity(int op);
template <> __device__ __forceinline__ float red_identity<float>(int op) {
  return op == MTFC_REDUCE_SUM ? 0.f : (op == MTFC_REDUCE_MAX ? -INFINITY : INFINITY);
}
template <> __device__ __forceinline__ int red_identity<int>(int op) {
  return op == MTFC_REDUCE_SUM ? 0 : (op == MTFC_REDUCE_MAX ? INT_MIN : INT_MAX);
}
template <typename C> __device__ __forceinline__ C red_combine(int op, C a, C b) {
  return op == MTFC_REDUCE_SUM ? a + b : (op == MTFC_REDUCE_MAX ? (a > b ? a : b) : (a < b ? a : b));
}

template <typename TI, typename TO, bool kWarp>
__global__ void broadcast_reduce_kernel(int op, int n_in, const TI* __restrict__ in0,
                                        const TI* __restrict__ in1, const TI* __restrict__ in2,
                                        const TI* __restrict__ in3, TO* __restrict__ out,
                                        Dims out_dims, Dims red_dims, long long n_out,
                                        long long n_red) {
  using C = typename Compute<TI>::type;
  const TI* ins[4] = {in0, in1, in2, in3};
  const int lane = threadIdx.x & 31;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long first = kWarp ? tid / 32 : tid;
  const long long step = kWarp ? nthreads / 32 : nthreads;
  for (long long o = first; o < n_out; o += step) {
    long long base[4] = {0, 0, 0, 0};
    long long rem = o;
#pragma unroll 1
    for (int d = out_dims.ndim - 1; d >= 0; --d) {
      const long long c = rem % out_dims.shape[d];
      rem /= out_dims.shape[d];
      for (int k = 0; k < n_in; ++k) base[k] += c * out_dims.stride[k][d];
    }
    C acc = red_identity<C>(op);
    for (long long r = kWarp ? lane : 0; r < n_red; r += kWarp ? 32 : 1) {
      long long off[4] = {base[0], base[1], base[2], base[3]};
      long long rr = r;
#pragma unroll 1
      for (int d = red_dims.ndim - 1; d >= 0; --d) {
        const long long c = rr % red_dims.shape[d];
        rr /= red_dims.shape[d];
        for (int k = 0; k < n_in; ++k) off[k] += c * red_dims.stride[k][d];
      }
      C v = ld<TI>(ins[0], off[0]);
      for (int k = 1; k < n_in; ++k) v = v * ld<TI>(ins[k], off[k]);
      acc = red_combine<C>(op, acc, v);
    }
    if (kWarp) {
#pragma unroll
      for (int s = 16; s > 0; s >>= 1)
        acc = red_combine<C>(op, acc, __shfl_xor_sync(0xffffffffu, acc, s));
      if (lane == 0) st<TO>(out, o, acc);
    } else {
      st<TO>(out, o, acc);
    }
  }
}

// ---------------------------------------------- arg-max / top-k / gather
// One thread per row; ties go to the lowest index.
template <typename T>
__global__ void topk_last_kernel(const T* __restrict__ x, long long rows, int cols, int k,
                                 T* __restrict__ values, int* __restrict__ indices) {
  using C = typename Compute<T>::type;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += step) {
    const T* row = x + r * cols;
    C last_v = 0;
    int last_i = -1;
    for (int j = 0; j < k; ++j) {
      // Next element in (value desc, index asc) order after (last_v, last_i).
      bool have = false;
      C best_v = 0;
      int best_i = 0;
      for (int c = 0; c < cols; ++c) {
        const C v = ld<T>(row, c);
        if (j > 0 && !(v < last_v || (v == last_v && c > last_i))) continue;
        if (!have || v > best_v) { have = true; best_v = v; best_i = c; }
      }
      if (values) st<T>(values, r * k + j, best_v);
      indices[r * k + j] = best_i;
      last_v = best_v;
      last_i = best_i;
    }
  }
}

template <typename T>
__global__ void gather_last_kernel(const T* __restrict__ values, const int* __restrict__ idx,
                                   long long rows, int cols, int k, T* __restrict__ out) {
  const long long n = rows * k;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    const long long r = i / k;
    const int c = idx[i];
    out[i] = (c >= 0 && c < cols) ? values[r * cols + c] : values[r * cols];
  }
}

template <typename TO>
__global__ void one_hot_kernel(const int* __restrict__ idx, long long n, int depth, float on,
                               float off, TO* __restrict__ out) {
  const long long total = n * depth;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
    const long long r = i / depth;
    const int c = (int)(i - r * depth);
    st<TO>(out, i, idx[r] == c ? on : off);
  }
}

template <typename TO>
__global__ void fill_kernel(TO* __restrict__ out, long long n, float value, float step_value) {
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step)
    st<TO>(out, i, value + step_value * (float)i);
}

// fp32 [batch, rows, k] (any strides) -> bf16 [batch, rows, 6k]: each value is
// split as hi + mid + lo (three bf16 terms carrying 24 mantissa bits) and the
// terms are laid along K in the order `pattern` names, so that one bf16 GEMM
// over 6k with fp32 accumulation sums hi*lo + lo*hi + mid*mid + hi*mid + mid*hi +
// hi*hi — every product exact in fp32 — i.e. an fp32-accurate contraction on
// the tensor cores.  The K blocks are ordered smallest products first: the
// tensor core truncates when it adds into the fp32 accumulator, so the many
// correction terms are added while the accumulator is still ~2^-8 of its final
// size and only the k/16 additions of the hi*hi block see its full magnitude.
// pattern 0 (left operand): hi lo mid hi mid hi;
// pattern 1 (right operand): lo hi mid mid hi hi.
__global__ void split_bf16x3_kernel(const float* __restrict__ src, long long s_batch,
                                    long long s_row, long long s_k, __nv_bfloat16* __restrict__ dst,
                                    long long batch, long long rows, long long k, int pattern) {
  const long long n = batch * rows * k;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    const long long kk = i % k;
    const long long r = (i / k) % rows;
    const long long b = i / (k * rows);
    const float v = src[b * s_batch + r * s_row + kk * s_k];
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    const __nv_bfloat16 lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
    __nv_bfloat16* o = dst + (b * rows + r) * 6 * k + kk;
    if (pattern == 0) {
      o[0] = hi; o[k] = lo; o[2 * k] = mid; o[3 * k] = hi; o[4 * k] = mid; o[5 * k] = hi;
    } else {
      o[0] = lo; o[k] = hi; o[2 * k] = mid; o[3 * k] = mid; o[4 * k] = hi; o[5 * k] = hi;
    }
  }
}

// ------------------------------------------------------------ host helpers
int fill_dims(Dims* d, int ndim, const int64_t* shape, const int64_t* const* strides, int n_str) {
  if (ndim < 0 || ndim > MTFC_MAX_DIMS) return fail(MTFC_ERR_SHAPE, "ndim %d out of range", ndim);
  d->ndim = ndim;
  for (int i = 0; i < MTFC_MAX_DIMS; ++i) {
    d->shape[i] = i < ndim ? shape[i] : 1;
    for (int k = 0; k < 4; ++k)
      d->stride[k][i] = (i < ndim && k < n_str && strides[k]) ? strides[k][i] : 0;
  }
  return MTFC_OK;
}

long long volume(int ndim, const int64_t* shape) {
  long long n = 1;
  for (int i = 0; i < ndim; ++i) n *= shape[i];
  return n;
}

#define DISPATCH_IN_OUT(in_dt, out_dt, EXPR)                                             \
  do {                                                                                   \
    if (in_dt == MTFC_F32 && out_dt == MTFC_F32) { using TI = float; using TO = float; EXPR; } \
    else if (in_dt == MTFC_F32 && out_dt == MTFC_BF16) { using TI = float; using TO = __nv_bfloat16; EXPR; } \
    else if (in_dt == MTFC_F32 && out_dt == MTFC_I32) { using TI = float; using TO = int; EXPR; } \
    else if (in_dt == MTFC_BF16 && out_dt == MTFC_F32) { using TI = __nv_bfloat16; using TO = float; EXPR; } \
    else if (in_dt == MTFC_BF16 && out_dt == MTFC_BF16) { using TI = __nv_bfloat16; using TO = __nv_bfloat16; EXPR; } \
    else if (in_dt == MTFC_BF16 && out_dt == MTFC_I32) { using TI = __nv_bfloat16; using TO = int; EXPR; } \
    else if (in_dt == MTFC_I32 && out_dt == MTFC_F32) { using TI = int; using TO = float; EXPR; } \
    else if (in_dt == MTFC_I32 && out_dt == MTFC_BF16) { using TI = int; using TO = __nv_bfloat16; EXPR; } \
    else if (in_dt == MTFC_I32 && out_dt == MTFC_I32) { using TI = int; using TO = int; EXPR; } \
    else return fail(MTFC_ERR_UNSUPPORTED, "dtype pair (%d,%d) not implemented", in_dt, out_dt); \
  } while (0)

#define DISPATCH_ONE(dt, EXPR)                                                  \
  do {                                                                          \
    if (dt == MTFC_F32) { using T = float; EXPR; }                              \
    else if (dt == MTFC_BF16) { using T = __nv_bfloat16; EXPR; }                \
    else if (dt == MTFC_I32) { using T = int; EXPR; }                           \
    else return fail(MTFC_ERR_UNSUPPORTED, "dtype %d not implemented", dt);     \
  } while (0)

}  // namespace
}  // namespace mtfc

using namespace mtfc;

extern "C" {

int mtfc_unary(int op, const void* x, int x_dtype, void* y, int y_dtype, int64_t n, void* stream) {
  if (n < 0 || (n > 0 && (!x || !y))) return fail(MTFC_ERR_SHAPE, "unary: bad arguments");
  if (n == 0) return MTFC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (x_dtype == y_dtype && aligned16_all(x, y, nullptr) && n >= 4096) {
    // 16-byte body, scalar tail
    DISPATCH_ONE(x_dtype, (launch_unary_vec<T>(op, x, y, n, s)));
    MTFC_LAUNCH_CHECK("unary_vec_kernel");
    count_launch(1);
    return MTFC_OK;
  }
  DISPATCH_IN_OUT(x_dtype, y_dtype,
                  (unary_kernel<TI, TO><<<grid_for(n, kThreads * 4), kThreads, 0, s>>>(
                      op, static_cast<const TI*>(x), static_cast<TO*>(y), n)));
  MTFC_LAUNCH_CHECK("unary_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_binary(int op, const void* a, const int64_t* a_strides, const void* b,
                const int64_t* b_strides, double scalar_b, void* out, int in_dtype,
                int out_dtype, int ndim, const int64_t* shape, void* stream) {
  if (!a || !out) return fail(MTFC_ERR_SHAPE, "binary: null argument");
  Dims dims;
  const int64_t* strides[2] = {a_strides, b_strides};
  int rc = fill_dims(&dims, ndim, shape, strides, 2);
  if (rc != MTFC_OK) return rc;
  const long long n = volume(ndim, shape);
  if (n == 0) return MTFC_OK;
  // contiguous same-shape operands take the flat path
  bool flat = true;
  long long expect = 1;
  for (int d = ndim - 1; d >= 0; --d) {
    if (shape[d] != 1) {
      if (a_strides[d] != expect) flat = false;
      if (b && b_strides[d] != expect) flat = false;
    }
    expect *= shape[d];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (flat && in_dtype == out_dtype && aligned16_all(a, b, out) && n >= 4096) {
    // 16-byte body, scalar tail
    DISPATCH_ONE(in_dtype, (launch_binary_vec<T>(op, a, b, scalar_b, out, n, s)));
  } else if (flat) {
    DISPATCH_IN_OUT(in_dtype, out_dtype,
                    (binary_flat_kernel<TI, TO><<<grid_for(n, kThreads * 4), kThreads, 0, s>>>(
                        op, static_cast<const TI*>(a), static_cast<const TI*>(b), scalar_b,
                        static_cast<TO*>(out), n)));
  } else {
    DISPATCH_IN_OUT(in_dtype, out_dtype,
                    (binary_kernel<TI, TO><<<grid_for(n, kThreads * 2), kThreads, 0, s>>>(
                        op, static_cast<const TI*>(a), static_cast<const TI*>(b), scalar_b,
                        static_cast<TO*>(out), dims, n)));
  }
  MTFC_LAUNCH_CHECK("binary_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_copy_strided(const void* src, const int64_t* src_strides, void* dst,
                      const int64_t* dst_strides, int ndim, const int64_t* shape, int elem_bytes,
                      void* stream) {
  if (elem_bytes != 2 && elem_bytes != 4)
    return fail(MTFC_ERR_UNSUPPORTED, "copy_strided: element size %d", elem_bytes);
  const long long n = volume(ndim, shape);
  if (n == 0) return MTFC_OK;
  if (!src || !dst) return fail(MTFC_ERR_SHAPE, "copy_strided: null argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Merge the trailing dims that are contiguous on both sides into one row.
  long long row = 1;
  int nd = ndim;
  while (nd > 0 && (shape[nd - 1] == 1 ||
                    (src_strides[nd - 1] == row && dst_strides[nd - 1] == row))) {
    row *= shape[nd - 1];
    --nd;
  }
  const long long row_bytes = row * elem_bytes;
  bool vec_ok = row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 &&
                reinterpret_cast<uintptr_t>(dst) % 16 == 0;
  for (int d = 0; d < nd && vec_ok; ++d)
    if ((src_strides[d] * elem_bytes) % 16 != 0 || (dst_strides[d] * elem_bytes) % 16 != 0)
      vec_ok = false;
  if (vec_ok) {
    Dims dims;
    int64_t ss[MTFC_MAX_DIMS], ds[MTFC_MAX_DIMS];
    for (int d = 0; d < nd; ++d) {
      ss[d] = src_strides[d] * elem_bytes / 16;
      ds[d] = dst_strides[d] * elem_bytes / 16;
    }
    const int64_t* strides[2] = {ss, ds};
    int rc = fill_dims(&dims, nd, shape, strides, 2);
    if (rc != MTFC_OK) return rc;
    const long long vec_per_row = row_bytes / 16;
    const long long n_vec = n * elem_bytes / 16;
    copy_rows16_kernel<<<grid_for(n_vec, kThreads * 2), kThreads, 0, s>>>(
        static_cast<const uint4*>(src), static_cast<uint4*>(dst), dims, vec_per_row, n_vec);
  } else {
    Dims dims;
    const int64_t* strides[2] = {src_strides, dst_strides};
    int rc = fill_dims(&dims, ndim, shape, strides, 2);
    if (rc != MTFC_OK) return rc;
    if (elem_bytes == 4)
      copy_strided_kernel<uint32_t><<<grid_for(n, kThreads * 2), kThreads, 0, s>>>(
          static_cast<const uint32_t*>(src), static_cast<uint32_t*>(dst), dims, n);
    else
      copy_strided_kernel<uint16_t><<<grid_for(n, kThreads * 2), kThreads, 0, s>>>(
          static_cast<const uint16_t*>(src), static_cast<uint16_t*>(dst), dims, n);
  }
  MTFC_LAUNCH_CHECK("copy_strided_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_broadcast_reduce(int op, int n_in, const void* const* in, int in_dtype, void* out,
                          int out_dtype, int ndim_out, const int64_t* out_shape,
                          const int64_t* const* out_strides, int ndim_red,
                          const int64_t* red_shape, const int64_t* const* red_strides,
                          void* stream) {
  if (n_in < 1 || n_in > 4) return fail(MTFC_ERR_SHAPE, "broadcast_reduce: %d operands", n_in);
  if (n_in > 1 && op != MTFC_REDUCE_SUM)
    return fail(MTFC_ERR_UNSUPPORTED, "broadcast_reduce: products reduce with SUM only");
  Dims od, rd;
  int rc = fill_dims(&od, ndim_out, out_shape, out_strides, n_in);
  if (rc != MTFC_OK) return rc;
  rc = fill_dims(&rd, ndim_red, red_shape, red_strides, n_in);
  if (rc != MTFC_OK) return rc;
  const long long n_out = volume(ndim_out, out_shape);
  const long long n_red = volume(ndim_red, red_shape);
  if (n_out == 0) return MTFC_OK;
  const void* p[4] = {in[0], n_in > 1 ? in[1] : nullptr, n_in > 2 ? in[2] : nullptr,
                      n_in > 3 ? in[3] : nullptr};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // A warp per output pays off once the reduced extent is long and there are
  // too few outputs to fill the machine with single threads.
  const bool warp = n_red >= 64 && n_out < (long long)sm_count() * 2048;
  if (warp) {
    DISPATCH_IN_OUT(in_dtype, out_dtype,
                    (broadcast_reduce_kernel<TI, TO, true>
                     <<<grid_for(n_out * 32, kThreads), kThreads, 0, s>>>(
                         op, n_in, static_cast<const TI*>(p[0]), static_cast<const TI*>(p[1]),
                         static_cast<const TI*>(p[2]), static_cast<const TI*>(p[3]),
                         static_cast<TO*>(out), od, rd, n_out, n_red)));
  } else {
    DISPATCH_IN_OUT(in_dtype, out_dtype,
                    (broadcast_reduce_kernel<TI, TO, false>
                     <<<grid_for(n_out, kThreads), kThreads, 0, s>>>(
                         op, n_in, static_cast<const TI*>(p[0]), static_cast<const TI*>(p[1]),
                         static_cast<const TI*>(p[2]), static_cast<const TI*>(p[3]),
                         static_cast<TO*>(out), od, rd, n_out, n_red)));
  }
  MTFC_LAUNCH_CHECK("broadcast_reduce_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_topk_last(const void* x, int dtype, int64_t rows, int32_t cols, int32_t k, void* values,
                   int32_t* indices, void* stream) {
  if (rows < 0 || cols < 1 || k < 1 || k > cols) return fail(MTFC_ERR_SHAPE, "topk: bad extents");
  if (rows == 0) return MTFC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  DISPATCH_ONE(dtype, (topk_last_kernel<T><<<grid_for(rows, 128), 128, 0, s>>>(
                          static_cast<const T*>(x), rows, cols, k, static_cast<T*>(values),
                          indices)));
  MTFC_LAUNCH_CHECK("topk_last_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_gather_last(const void* values, int dtype, const int32_t* indices, int64_t rows,
                     int32_t cols, int32_t k, void* out, void* stream) {
  if (rows < 0 || cols < 1 || k < 1) return fail(MTFC_ERR_SHAPE, "gather: bad extents");
  if (rows == 0) return MTFC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  DISPATCH_ONE(dtype, (gather_last_kernel<T><<<grid_for(rows * k, kThreads), kThreads, 0, s>>>(
                          static_cast<const T*>(values), indices, rows, cols, k,
                          static_cast<T*>(out))));
  MTFC_LAUNCH_CHECK("gather_last_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_one_hot(const int32_t* indices, int64_t n, int32_t depth, float on_value,
                 float off_value, void* out, int out_dtype, void* stream) {
  if (n < 0 || depth < 0) return fail(MTFC_ERR_SHAPE, "one_hot: bad extents");
  if (n == 0 || depth == 0) return MTFC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  DISPATCH_ONE(out_dtype, (one_hot_kernel<T><<<grid_for(n * depth, kThreads * 4), kThreads, 0, s>>>(
                              indices, n, depth, on_value, off_value, static_cast<T*>(out))));
  MTFC_LAUNCH_CHECK("one_hot_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_fill(void* out, int dtype, int64_t n, float value, float step, void* stream) {
  if (n < 0) return fail(MTFC_ERR_SHAPE, "fill: negative size");
  if (n == 0) return MTFC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  DISPATCH_ONE(dtype, (fill_kernel<T><<<grid_for(n, kThreads * 4), kThreads, 0, s>>>(
                          static_cast<T*>(out), n, value, step)));
  MTFC_LAUNCH_CHECK("fill_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_split_bf16x3(const float* src, int64_t s_batch, int64_t s_row, int64_t s_k, void* dst_bf16,
                      int64_t batch, int64_t rows, int64_t k, int pattern, void* stream) {
  if (batch < 0 || rows < 0 || k < 0 || (pattern != 0 && pattern != 1))
    return fail(MTFC_ERR_SHAPE, "split_bf16x3: bad arguments");
  const long long n = batch * rows * k;
  if (n == 0) return MTFC_OK;
  if (!src || !dst_bf16) return fail(MTFC_ERR_SHAPE, "split_bf16x3: null argument");
  split_bf16x3_kernel<<<grid_for(n, kThreads * 2), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      src, s_batch, s_row, s_k, static_cast<__nv_bfloat16*>(dst_bf16), batch, rows, k, pattern);
  MTFC_LAUNCH_CHECK("split_bf16x3_kernel");
  count_launch(1);
  return MTFC_OK;
}

}  // extern "C"
