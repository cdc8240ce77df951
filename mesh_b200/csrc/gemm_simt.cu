// K1f: strided batched contraction on the FFMA pipes.
//
// C[b,m,n] = epilogue(sum_k A[b,m,k] * B[b,k,n]) for operands the tensor-core
// kernel does not take: fp32 (the 1e-5 tolerance of fp32 einsums rules out a
// single-pass bf16/tf32 MMA), int32, and bf16 with strides a TMA tensor map
// cannot describe.  Replaces the same tf.einsum call as the tensor-core kernel
// (mesh_tensorflow/ops.py:1331-1340, 2816-2822).  All nine strides are free,
// so any named-dim order is read in place; accumulation is fp32 (int32 for
// integer operands) with one rounding at the store.
//
// 128x128x16 tiles, 256 threads, 8x8 outputs per thread; global loads are
// ordered along whichever stride of each operand is 1 so they coalesce.

#include "common.cuh"

namespace mtfc {
namespace {

constexpr int TM = 128, TN = 128, TK = 16;
constexpr int PAD = 4;

template <typename T> struct Acc { using type = float; };
template <> struct Acc<int> { using type = int; };

template <typename T> __device__ __forceinline__ typename Acc<T>::type widen(T v);
template <> __device__ __forceinline__ float widen<float>(float v) { return v; }
template <> __device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <> __device__ __forceinline__ int widen<int>(int v) { return v; }

template <typename TO, typename TA> __device__ __forceinline__ TO narrow(TA v);
template <> __device__ __forceinline__ float narrow<float, float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16, float>(float v) {
  return __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ int narrow<int, float>(float v) { return (int)v; }
template <> __device__ __forceinline__ int narrow<int, int>(int v) { return v; }
template <> __device__ __forceinline__ float narrow<float, int>(int v) { return (float)v; }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16, int>(int v) {
  return __float2bfloat16_rn((float)v);
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TI* __restrict__ A, const TI* __restrict__ B, TO* __restrict__ C,
                 mtfc_gemm_desc d, int tiles_m, int tiles_n) {
  using TA = typename Acc<TI>::type;
  __shared__ TA As[TK][TM + PAD];
  __shared__ TA Bs[TK][TN + PAD];

  const long long tiles_per_batch = (long long)tiles_m * tiles_n;
  const long long num_tiles = tiles_per_batch * d.batch;
  const int tid = threadIdx.x;
  const int tx = tid & 15;  // n direction
  const int ty = tid >> 4;  // m direction
  const bool a_k_fast = (d.a_k == 1) || (d.a_m != 1);
  const bool b_n_fast = (d.b_n == 1) || (d.b_k != 1);

  for (long long t = blockIdx.x; t < num_tiles; t += gridDim.x) {
    const long long b = t / tiles_per_batch;
    const int r = (int)(t % tiles_per_batch);
    const long long m0 = (long long)(r / tiles_n) * TM;
    const long long n0 = (long long)(r % tiles_n) * TN;
    const TI* Ab = A + b * d.a_batch;
    const TI* Bb = B + b * d.b_batch;

    TA acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = 0;

    for (long long k0 = 0; k0 < d.k; k0 += TK) {
#pragma unroll
      for (int i = 0; i < (TM * TK) / 256; ++i) {
        const int idx = tid + i * 256;
        int mm, kk;
        if (a_k_fast) { kk = idx % TK; mm = idx / TK; } else { mm = idx % TM; kk = idx / TM; }
        const long long gm = m0 + mm, gk = k0 + kk;
        TA v = 0;
        if (gm < d.m && gk < d.k) v = widen<TI>(Ab[gm * d.a_m + gk * d.a_k]);
        As[kk][mm] = v;
      }
#pragma unroll
      for (int i = 0; i < (TN * TK) / 256; ++i) {
        const int idx = tid + i * 256;
        int nn, kk;
        if (b_n_fast) { nn = idx % TN; kk = idx / TN; } else { kk = idx % TK; nn = idx / TK; }
        const long long gn = n0 + nn, gk = k0 + kk;
        TA v = 0;
        if (gn < d.n && gk < d.k) v = widen<TI>(Bb[gk * d.b_k + gn * d.b_n]);
        Bs[kk][nn] = v;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < TK; ++kk) {
        TA a[8], bv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = As[kk][ty * 4 + (i & 3) + (i >> 2) * 64];
#pragma unroll
        for (int j = 0; j < 8; ++j) bv[j] = Bs[kk][tx * 4 + (j & 3) + (j >> 2) * 64];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] += a[i] * bv[j];
      }
      __syncthreads();
    }

    TO* Cb = C + b * d.c_batch;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const long long gm = m0 + ty * 4 + (i & 3) + (i >> 2) * 64;
      if (gm >= d.m) continue;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const long long gn = n0 + tx * 4 + (j & 3) + (j >> 2) * 64;
        if (gn >= d.n) continue;
        TA v = acc[i][j];
        if (d.epilogue == MTFC_EPILOGUE_RELU) v = v > 0 ? v : 0;
        Cb[gm * d.c_m + gn * d.c_n] = narrow<TO, TA>(v);
      }
    }
  }
}

template <typename TI, typename TO>
int launch(const mtfc_gemm_desc* d, const void* a, const void* b, void* c, cudaStream_t stream) {
  const int tiles_m = (int)((d->m + TM - 1) / TM);
  const int tiles_n = (int)((d->n + TN - 1) / TN);
  const long long tiles = (long long)tiles_m * tiles_n * d->batch;
  const long long cap = (long long)sm_count() * 2;
  const unsigned grid = (unsigned)(tiles < cap ? tiles : cap);
  gemm_simt_kernel<TI, TO><<<grid, 256, 0, stream>>>(
      static_cast<const TI*>(a), static_cast<const TI*>(b), static_cast<TO*>(c), *d, tiles_m,
      tiles_n);
  MTFC_LAUNCH_CHECK("gemm_simt_kernel");
  return MTFC_OK;
}

}  // namespace

int gemm_simt_launch(const mtfc_gemm_desc* d, const void* a, const void* b, void* c,
                     cudaStream_t stream) {
  const int in = d->in_dtype, out = d->out_dtype;
  if (in == MTFC_F32 && out == MTFC_F32) return launch<float, float>(d, a, b, c, stream);
  if (in == MTFC_F32 && out == MTFC_BF16) return launch<float, __nv_bfloat16>(d, a, b, c, stream);
  if (in == MTFC_BF16 && out == MTFC_BF16)
    return launch<__nv_bfloat16, __nv_bfloat16>(d, a, b, c, stream);
  if (in == MTFC_BF16 && out == MTFC_F32) return launch<__nv_bfloat16, float>(d, a, b, c, stream);
  if (in == MTFC_I32 && out == MTFC_I32) return launch<int, int>(d, a, b, c, stream);
  if (in == MTFC_I32 && out == MTFC_F32) return launch<int, float>(d, a, b, c, stream);
  return fail(MTFC_ERR_UNSUPPORTED, "gemm: in_dtype %d -> out_dtype %d not implemented", in, out);
}

}  // namespace mtfc
