// K2-K5: top-2 mixture-of-experts routing as scan / gather / scatter kernels.
//
// These replace the op chain of `_top_2_gating`
// (mesh_tensorflow/transformer/moe.py:1380-1513) and the two dense one-hot
// einsums around the experts (moe.py:443-447 dispatch, 509-510 combine):
//
//   split_gate_weights : fp32 gate kernel -> three bf16 terms [M, 3E] so the
//                        gate logits can be formed on the tensor cores with
//                        fp32-level accuracy (activations are bf16, hence
//                        exact; each bf16 x bf16 product is exact in fp32)
//   top2_gating        : one CTA per group. logits -> softmax in the
//                        exp(x - logsumexp) form -> top-1 -> masked top-2 ->
//                        renormalised gates -> second-expert policy ->
//                        position-in-expert by warp match/popc scans carried
//                        across token chunks -> capacity masks -> per-group
//                        load-balancing loss.  Token order within a group is
//                        index order, ties go to the lowest expert index.
//   slot_table         : (expert, slot) -> token map of a group (-1 = empty)
//   dispatch_rows      : expert_inputs[E,G,C,M] row gather, zero rows for
//                        empty slots, every output row written exactly once
//   combine_rows       : out[g,s,:] = w1 * y[i1,g,p1,:] + w2 * y[i2,g,p2,:]
//
// Gating is latency/HBM-light; dispatch and combine are HBM-bound 16-byte
// vector row copies with one warp per row.

#include "common.cuh"

namespace mtfc {
namespace {

constexpr int kMaxExperts = 256;
constexpr int kGateSegments = 32;  // row segments of the per-expert column sums

__global__ void split_gate_weights_kernel(const float* __restrict__ w, long long m, int e,
                                          __nv_bfloat16* __restrict__ out) {
  const long long n = m * e;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    const long long row = i / e;
    const int col = (int)(i - row * e);
    const float v = w[i];
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(hi);
    const __nv_bfloat16 mid = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(mid);
    const __nv_bfloat16 lo = __float2bfloat16_rn(r2);
    __nv_bfloat16* o = out + row * 3 * e;
    o[col] = hi;
    o[e + col] = mid;
    o[2 * e + col] = lo;
  }
}

__device__ __forceinline__ bool bf16_nonzero(float g) {
  return __bfloat162float(__float2bfloat16_rn(g)) != 0.0f;
}

struct GateArgs {
  const float* logits;  // [groups * group_size, parts * experts]
  int parts;
  int group_size, experts, capacity;
  int policy;
  float threshold;
  const float* noise;  // [groups * group_size] or null
  int* idx1;
  int* idx2;
  int* pos1;
  int* pos2;
  float* gate1;
  float* gate2;
  float* raw_gates;       // [groups * group_size, experts] or null
  float* loss_per_group;  // [groups]
};

// One CTA of T = blockDim.x threads per group; tokens are taken T at a time.
// Dynamic shared memory layout (floats / ints):
//   row   [T][experts + 1]             logits then raw gates of the chunk
//   proxy [experts]                    running sum over tokens of raw gates
//   part  [kGateSegments][experts]     partial column sums (fixed order: deterministic)
//   base1 [experts], base2 [experts]   running per-expert counts (1st / 2nd)
//   wcnt  [T / 32][experts]            per-warp counts of the chunk
//   cnt1  [experts]                    kept first-choice count
__global__ void __launch_bounds__(1024)
top2_gating_kernel(GateArgs a) {
  extern __shared__ float smem[];
  const int E = a.experts;
  const int S = a.group_size;
  const int ld = E + 1;
  const int kGateThreads = blockDim.x;
  const int kGateWarps = kGateThreads >> 5;
  float* row = smem;
  float* proxy = row + kGateThreads * ld;
  float* part = proxy + E;
  int* base1 = reinterpret_cast<int*>(part + kGateSegments * E);
  int* base2 = base1 + E;
  int* wcnt = base2 + E;
  int* cnt1 = wcnt + kGateWarps * E;

  const int g = blockIdx.x;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const unsigned lt_mask = (1u << lane) - 1u;
  const long long tok0 = (long long)g * S;

  for (int e = tid; e < E; e += kGateThreads) { proxy[e] = 0.f; base1[e] = 0; base2[e] = 0; }
  __syncthreads();

  // ---- pass 1: softmax, top-2, gates, first-choice positions ----
  for (int c0 = 0; c0 < S; c0 += kGateThreads) {
    const int chunk = min(kGateThreads, S - c0);
    // cooperative, coalesced load of the chunk's logits, summing the parts
    const int width = a.parts * E;
    const float* src = a.logits + (tok0 + c0) * width;
    for (int i = tid; i < chunk * E; i += kGateThreads) {
      const int t = i / E, e = i - t * E;
      float v = src[(long long)t * width + e];
      for (int p = 1; p < a.parts; ++p) v += src[(long long)t * width + p * E + e];
      row[t * ld + e] = v;
    }
    for (int i = tid; i < kGateWarps * E; i += kGateThreads) wcnt[i] = 0;
    __syncthreads();

    const bool live = tid < chunk;
    int i1 = -1, i2 = -1;
    float g1 = 0.f, g2 = 0.f;
    if (live) {
      float* r = row + tid * ld;
      float mx = r[0];
      for (int e = 1; e < E; ++e) mx = fmaxf(mx, r[e]);
      float sum = 0.f;
      for (int e = 0; e < E; ++e) sum += expf(r[e] - mx);
      const float lse = logf(sum) + mx;
      float b1 = -1.f;
      for (int e = 0; e < E; ++e) {
        const float p = expf(r[e] - lse);
        r[e] = p;
        if (p > b1) { b1 = p; i1 = e; }
      }
      float b2 = -1.f;
      for (int e = 0; e < E; ++e) {
        const float p = (e == i1) ? 0.f : r[e];
        if (p > b2) { b2 = p; i2 = e; }
      }
      const float denom = (b1 + b2) + 1e-9f;
      const float recip = 1.0f / denom;
      g1 = a.policy == MTFC_MOE_POLICY_SWITCH ? b1 : b1 * recip;
      g2 = a.policy == MTFC_MOE_POLICY_SWITCH ? 0.f : b2 * recip;
      if (a.raw_gates) {
        float* dst = a.raw_gates + (tok0 + c0 + tid) * E;
        for (int e = 0; e < E; ++e) dst[e] = r[e];
      }
    }
    // first-choice rank inside the warp, per-warp counts
    const unsigned same = __match_any_sync(0xffffffffu, i1);
    const int rank = __popc(same & lt_mask);
    if (live && rank == 0) wcnt[warp * E + i1] = __popc(same);
    __syncthreads();
    // column sums of the raw gates for the loss: kGateSegments partial sums per
    // expert, combined in a fixed order below
    {
      const int rows_per_seg = (chunk + kGateSegments - 1) / kGateSegments;
      for (int i = tid; i < kGateSegments * E; i += kGateThreads) {
        const int seg = i / E, e = i - seg * E;
        const int r0 = seg * rows_per_seg;
        const int r1 = min(chunk, r0 + rows_per_seg);
        float s = 0.f;
        for (int t = r0; t < r1; ++t) s += row[t * ld + e];
        part[seg * E + e] = s;
      }
    }
    __syncthreads();
    // cross-warp offsets of the first-choice counts
    for (int e = tid; e < E; e += kGateThreads) {
      float s = 0.f;
      for (int seg = 0; seg < kGateSegments; ++seg) s += part[seg * E + e];
      proxy[e] += s;
      int run = base1[e];
      for (int w = 0; w < kGateWarps; ++w) {
        const int c = wcnt[w * E + e];
        wcnt[w * E + e] = run;
        run += c;
      }
      base1[e] = run;
    }
    __syncthreads();
    if (live) {
      const long long t = tok0 + c0 + tid;
      a.idx1[t] = i1;
      a.idx2[t] = i2;
      a.pos1[t] = wcnt[warp * E + i1] + rank;
      a.gate1[t] = g1;
      a.gate2[t] = g2;
    }
    __syncthreads();
  }

  // ---- loss and first-choice kept counts ----
  for (int e = tid; e < E; e += kGateThreads) cnt1[e] = min(base1[e], a.capacity);
  __syncthreads();
  if (warp == 0) {
    float part = 0.f;
    const float inv_s = 1.0f / (float)S;
    for (int e = lane; e < E; e += 32)
      part += (proxy[e] * inv_s) * ((float)base1[e] * inv_s);
    for (int s = 16; s > 0; s >>= 1) part += __shfl_xor_sync(0xffffffffu, part, s);
    if (lane == 0) a.loss_per_group[g] = part * (1.0f / (float)E) * (float)(E * E);
  }

  // ---- pass 2: second-choice policy, positions, capacity masks ----
  for (int c0 = 0; c0 < S; c0 += kGateThreads) {
    const int chunk = min(kGateThreads, S - c0);
    for (int i = tid; i < kGateWarps * E; i += kGateThreads) wcnt[i] = 0;
    __syncthreads();
    const bool live = tid < chunk;
    const long long t = tok0 + c0 + tid;
    int i2 = -1 - lane;  // dead lanes never match a live expert index
    float g1 = 0.f, g2 = 0.f;
    int p1 = 0;
    bool m2 = false;
    if (live) {
      g1 = a.gate1[t];
      g2 = a.gate2[t];
      p1 = a.pos1[t];
      const int cand = a.idx2[t];
      switch (a.policy) {
        case MTFC_MOE_POLICY_ALL: m2 = true; break;
        case MTFC_MOE_POLICY_NONE: m2 = false; break;
        case MTFC_MOE_POLICY_SWITCH: m2 = false; break;
        case MTFC_MOE_POLICY_THRESHOLD: m2 = g2 > a.threshold; break;
        case MTFC_MOE_POLICY_RANDOM:
          m2 = a.noise[t] < g2 * (1.0f / fmaxf(a.threshold, 1e-9f));
          break;
        default: m2 = true;
      }
      if (m2) i2 = cand;
    }
    const unsigned same = __match_any_sync(0xffffffffu, i2);
    const int rank = __popc(same & lt_mask);
    if (live && m2 && rank == 0) wcnt[warp * E + i2] = __popc(same);
    __syncthreads();
    for (int e = tid; e < E; e += kGateThreads) {
      int run = base2[e];
      for (int w = 0; w < kGateWarps; ++w) {
        const int c = wcnt[w * E + e];
        wcnt[w * E + e] = run;
        run += c;
      }
      base2[e] = run;
    }
    __syncthreads();
    if (live) {
      int p2 = 0;
      if (m2) p2 = wcnt[warp * E + i2] + rank + cnt1[i2];
      const bool keep1 = p1 < a.capacity;
      const bool keep2 = m2 && p2 < a.capacity;
      a.pos2[t] = p2;
      a.gate1[t] = keep1 ? g1 : 0.f;
      a.gate2[t] = keep2 ? g2 : 0.f;
    }
    __syncthreads();
  }
}

// (expert, slot) -> token of one group; -1 where no token was routed.
__global__ void __launch_bounds__(256)
slot_table_kernel(const int* __restrict__ idx1, const int* __restrict__ idx2,
                  const int* __restrict__ pos1, const int* __restrict__ pos2,
                  const float* __restrict__ gate1, const float* __restrict__ gate2, int S, int E,
                  int C, int round_bf16, int in_smem, int* __restrict__ table) {
  extern __shared__ int slots_smem[];
  const int g = blockIdx.x;
  const int n = E * C;
  // built in shared memory when the group's table fits there, else in place
  int* slots = in_smem ? slots_smem : table + (long long)g * n;
  for (int i = threadIdx.x; i < n; i += blockDim.x) slots[i] = -1;
  __syncthreads();
  const long long tok0 = (long long)g * S;
  for (int s = threadIdx.x; s < S; s += blockDim.x) {
    const long long t = tok0 + s;
    const float w1 = gate1[t], w2 = gate2[t];
    const int p1 = pos1[t], p2 = pos2[t];
    const int e1 = idx1[t], e2 = idx2[t];
    const bool k1 = (round_bf16 ? bf16_nonzero(w1) : w1 != 0.f) && p1 >= 0 && p1 < C &&
                    e1 >= 0 && e1 < E;
    const bool k2 = (round_bf16 ? bf16_nonzero(w2) : w2 != 0.f) && p2 >= 0 && p2 < C &&
                    e2 >= 0 && e2 < E;
    if (k1) slots[e1 * C + p1] = s;
    if (k2) slots[e2 * C + p2] = s;
  }
  __syncthreads();
  if (in_smem)
    for (int i = threadIdx.x; i < n; i += blockDim.x) table[(long long)g * n + i] = slots[i];
}

// out rows are [E][G][C] (slice layout [O=1 folded into G]); one warp per row.
__global__ void __launch_bounds__(256)
dispatch_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ table,
                     uint4* __restrict__ out, long long groups, int S, int E, int C,
                     int vec_per_row, long long og_stride_groups) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long rows = groups * E * C;
  for (long long r = warp; r < rows; r += nwarps) {
    // r enumerates output rows in [outer][E][G_inner][C] order
    const int c = (int)(r % C);
    long long rest = r / C;
    const long long gi = rest % og_stride_groups;
    rest /= og_stride_groups;
    const int e = (int)(rest % E);
    const long long o = rest / E;
    const long long g = o * og_stride_groups + gi;
    const int s = table[(g * E + e) * C + c];
    uint4* dst = out + r * vec_per_row;
    if (s >= 0) {
      const uint4* src = x + (g * S + s) * vec_per_row;
      for (int v = lane; v < vec_per_row; v += 32) dst[v] = src[v];
    } else {
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int v = lane; v < vec_per_row; v += 32) dst[v] = z;
    }
  }
}

template <typename T> struct Vec8;  // 16 bytes of T

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// y rows are [outer][E][G_inner][C]; out rows are tokens [G][S]; bf16 data.
__global__ void __launch_bounds__(256)
combine_rows_bf16_kernel(const uint4* __restrict__ y, const int* __restrict__ idx1,
                         const int* __restrict__ idx2, const int* __restrict__ pos1,
                         const int* __restrict__ pos2, const float* __restrict__ gate1,
                         const float* __restrict__ gate2, uint4* __restrict__ out,
                         long long groups, int S, int E, int C, int vec_per_row,
                         long long og_stride_groups) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long tokens = groups * S;
  for (long long t = warp; t < tokens; t += nwarps) {
    const long long g = t / S;
    const long long o = g / og_stride_groups, gi = g % og_stride_groups;
    const float w1 = __bfloat162float(__float2bfloat16_rn(gate1[t]));
    const float w2 = __bfloat162float(__float2bfloat16_rn(gate2[t]));
    const int p1 = pos1[t], p2 = pos2[t];
    const int e1 = idx1[t], e2 = idx2[t];
    const bool k1 = w1 != 0.f && p1 >= 0 && p1 < C && e1 >= 0 && e1 < E;
    const bool k2 = w2 != 0.f && p2 >= 0 && p2 < C && e2 >= 0 && e2 < E;
    const uint4* r1 = y + (((o * E + e1) * og_stride_groups + gi) * C + p1) * vec_per_row;
    const uint4* r2 = y + (((o * E + e2) * og_stride_groups + gi) * C + p2) * vec_per_row;
    uint4* dst = out + t * vec_per_row;
    for (int v = lane; v < vec_per_row; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (k1) {
        float f[8];
        unpack8(r1[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = w1 * f[i];
      }
      if (k2) {
        float f[8];
        unpack8(r2[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(w2, f[i], acc[i]);
      }
      dst[v] = pack8(acc);
    }
  }
}

__global__ void __launch_bounds__(256)
combine_rows_f32_kernel(const float4* __restrict__ y, const int* __restrict__ idx1,
                        const int* __restrict__ idx2, const int* __restrict__ pos1,
                        const int* __restrict__ pos2, const float* __restrict__ gate1,
                        const float* __restrict__ gate2, float4* __restrict__ out,
                        long long groups, int S, int E, int C, int vec_per_row,
                        long long og_stride_groups) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long tokens = groups * S;
  for (long long t = warp; t < tokens; t += nwarps) {
    const long long g = t / S;
    const long long o = g / og_stride_groups, gi = g % og_stride_groups;
    const float w1 = gate1[t], w2 = gate2[t];
    const int p1 = pos1[t], p2 = pos2[t];
    const int e1 = idx1[t], e2 = idx2[t];
    const bool k1 = w1 != 0.f && p1 >= 0 && p1 < C && e1 >= 0 && e1 < E;
    const bool k2 = w2 != 0.f && p2 >= 0 && p2 < C && e2 >= 0 && e2 < E;
    const float4* r1 = y + (((o * E + e1) * og_stride_groups + gi) * C + p1) * vec_per_row;
    const float4* r2 = y + (((o * E + e2) * og_stride_groups + gi) * C + p2) * vec_per_row;
    float4* dst = out + t * vec_per_row;
    for (int v = lane; v < vec_per_row; v += 32) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (k1) {
        const float4 f = r1[v];
        acc.x = w1 * f.x; acc.y = w1 * f.y; acc.z = w1 * f.z; acc.w = w1 * f.w;
      }
      if (k2) {
        const float4 f = r2[v];
        acc.x = fmaf(w2, f.x, acc.x); acc.y = fmaf(w2, f.y, acc.y);
        acc.z = fmaf(w2, f.z, acc.z); acc.w = fmaf(w2, f.w, acc.w);
      }
      dst[v] = acc;
    }
  }
}

// Backward of combine with respect to the expert outputs: slot (e, g, c) of dy
// receives w * dout[token of the slot], w being the gate (rounded to the data
// type, as in the forward pass) of the choice that put the token there.  Same
// traversal as dispatch_rows; empty slots get zero rows.
template <bool BF16>
__global__ void __launch_bounds__(256)
dispatch_rows_weighted_kernel(const uint4* __restrict__ x, const int* __restrict__ table,
                              const int* __restrict__ idx1, const int* __restrict__ pos1,
                              const float* __restrict__ gate1, const float* __restrict__ gate2,
                              uint4* __restrict__ out, long long groups, int S, int E, int C,
                              int vec_per_row, long long og_stride_groups) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long rows = groups * E * C;
  for (long long r = warp; r < rows; r += nwarps) {
    const int c = (int)(r % C);
    long long rest = r / C;
    const long long gi = rest % og_stride_groups;
    rest /= og_stride_groups;
    const int e = (int)(rest % E);
    const long long o = rest / E;
    const long long g = o * og_stride_groups + gi;
    const int s = table[(g * E + e) * C + c];
    uint4* dst = out + r * vec_per_row;
    if (s >= 0) {
      const long long t = g * S + s;
      const bool first = idx1[t] == e && pos1[t] == c && gate1[t] != 0.f;
      float w = first ? gate1[t] : gate2[t];
      if (BF16) w = __bfloat162float(__float2bfloat16_rn(w));
      const uint4* src = x + t * vec_per_row;
      for (int v = lane; v < vec_per_row; v += 32) {
        if (BF16) {
          float f[8];
          unpack8(src[v], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] *= w;
          dst[v] = pack8(f);
        } else {
          float4 f = reinterpret_cast<const float4*>(src)[v];
          f.x *= w; f.y *= w; f.z *= w; f.w *= w;
          reinterpret_cast<float4*>(dst)[v] = f;
        }
      }
    } else {
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int v = lane; v < vec_per_row; v += 32) dst[v] = z;
    }
  }
}

// Backward of combine with respect to the gates: dgate_k[t] = <dout[t, :], y[slot_k(t), :]>
// for the kept choices, 0 for the dropped ones.  One warp per token, fp32 sums.
template <bool BF16>
__global__ void __launch_bounds__(256)
combine_gate_grad_kernel(const uint4* __restrict__ y, const uint4* __restrict__ dout,
                         const int* __restrict__ idx1, const int* __restrict__ idx2,
                         const int* __restrict__ pos1, const int* __restrict__ pos2,
                         const float* __restrict__ gate1, const float* __restrict__ gate2,
                         float* __restrict__ dgate1, float* __restrict__ dgate2, long long groups,
                         int S, int E, int C, int vec_per_row, long long og_stride_groups) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const long long tokens = groups * S;
  for (long long t = warp; t < tokens; t += nwarps) {
    const long long g = t / S;
    const long long o = g / og_stride_groups, gi = g % og_stride_groups;
    float w1 = gate1[t], w2 = gate2[t];
    if (BF16) {
      w1 = __bfloat162float(__float2bfloat16_rn(w1));
      w2 = __bfloat162float(__float2bfloat16_rn(w2));
    }
    const int p1 = pos1[t], p2 = pos2[t];
    const int e1 = idx1[t], e2 = idx2[t];
    const bool k1 = w1 != 0.f && p1 >= 0 && p1 < C && e1 >= 0 && e1 < E;
    const bool k2 = w2 != 0.f && p2 >= 0 && p2 < C && e2 >= 0 && e2 < E;
    const uint4* r1 = y + (((o * E + e1) * og_stride_groups + gi) * C + p1) * vec_per_row;
    const uint4* r2 = y + (((o * E + e2) * og_stride_groups + gi) * C + p2) * vec_per_row;
    const uint4* d = dout + t * vec_per_row;
    float a1 = 0.f, a2 = 0.f;
    for (int v = lane; v < vec_per_row; v += 32) {
      if (BF16) {
        float dv[8];
        unpack8(d[v], dv);
        if (k1) {
          float f[8];
          unpack8(r1[v], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) a1 = fmaf(dv[i], f[i], a1);
        }
        if (k2) {
          float f[8];
          unpack8(r2[v], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) a2 = fmaf(dv[i], f[i], a2);
        }
      } else {
        const float4 dv = reinterpret_cast<const float4*>(d)[v];
        if (k1) {
          const float4 f = reinterpret_cast<const float4*>(r1)[v];
          a1 += dv.x * f.x + dv.y * f.y + dv.z * f.z + dv.w * f.w;
        }
        if (k2) {
          const float4 f = reinterpret_cast<const float4*>(r2)[v];
          a2 += dv.x * f.x + dv.y * f.y + dv.z * f.z + dv.w * f.w;
        }
      }
    }
    for (int sft = 16; sft > 0; sft >>= 1) {
      a1 += __shfl_xor_sync(0xffffffffu, a1, sft);
      a2 += __shfl_xor_sync(0xffffffffu, a2, sft);
    }
    if (lane == 0) {
      dgate1[t] = k1 ? a1 : 0.f;
      dgate2[t] = k2 ? a2 : 0.f;
    }
  }
}

// Slot-table scratch of mtfc_moe_dispatch_noalloc.  Lives in the library image:
// every GPU that loads libmtfc holds these 4 MiB until the process exits.
constexpr long long kNoAllocSlotCapacity = 1LL << 20;  // (group, expert, slot) entries
static __device__ __align__(256) int g_noalloc_slot_table[kNoAllocSlotCapacity];

// Device address of the scratch array on the current device.  The array's name
// is only a host-side handle here; kernels must be given the address the
// runtime resolves for the device that is current.
int noalloc_slot_table_ptr(int** out) {
  static int* ptrs[64] = {nullptr};
  int dev = 0;
  MTFC_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(MTFC_ERR_CUDA, "device ordinal %d out of range", dev);
  if (!ptrs[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_slot_table);
    if (e != cudaSuccess || !p)
      return fail(MTFC_ERR_CUDA, "cudaGetSymbolAddress(slot table scratch): %s",
                  cudaGetErrorString(e));
    ptrs[dev] = static_cast<int*>(p);
  }
  *out = ptrs[dev];
  return MTFC_OK;
}

size_t gate_smem_bytes(int experts, int threads) {
  return (size_t)(threads * (experts + 1) + experts + kGateSegments * experts) * sizeof(float) +
         (size_t)(3 * experts + (threads / 32) * experts) * sizeof(int);
}

// Largest power-of-two block (<= 1024, <= the group rounded up to a warp) whose
// chunk of logits fits in shared memory.
int gate_threads(int experts, int group_size) {
  int t = 1024;
  while (t > 32 && (gate_smem_bytes(experts, t) > 200 * 1024 || t / 2 >= group_size)) t >>= 1;
  return t;
}

}  // namespace
}  // namespace mtfc

using namespace mtfc;

extern "C" {

int mtfc_moe_split_gate_weights(const float* w, int64_t m, int32_t experts, void* out_bf16,
                                void* stream) {
  if (!w || !out_bf16 || m < 1 || experts < 1) return fail(MTFC_ERR_SHAPE, "split_gate_weights: bad arguments");
  const long long n = (long long)m * experts;
  split_gate_weights_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      w, m, experts, static_cast<__nv_bfloat16*>(out_bf16));
  MTFC_LAUNCH_CHECK("split_gate_weights_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_moe_top2_gating(const float* logits, int32_t parts, int64_t groups, int32_t group_size,
                         int32_t experts, int32_t capacity, int32_t policy, float threshold,
                         const float* noise, int32_t* idx1, int32_t* idx2, int32_t* pos1,
                         int32_t* pos2, float* gate1, float* gate2, float* raw_gates,
                         float* loss_per_group, void* stream) {
  if (!logits || !idx1 || !idx2 || !pos1 || !pos2 || !gate1 || !gate2 || !loss_per_group)
    return fail(MTFC_ERR_SHAPE, "top2_gating: null argument");
  if (groups < 0 || group_size < 1 || parts < 1 || capacity < 0)
    return fail(MTFC_ERR_SHAPE, "top2_gating: bad extents");
  if (experts < 2 || experts > kMaxExperts)
    return fail(MTFC_ERR_SHAPE, "top2_gating: experts=%d outside [2, %d]", experts, kMaxExperts);
  if (policy == MTFC_MOE_POLICY_RANDOM && !noise)
    return fail(MTFC_ERR_SHAPE, "top2_gating: policy random needs the noise tensor");
  if (policy < MTFC_MOE_POLICY_ALL || policy > MTFC_MOE_POLICY_SWITCH)
    return fail(MTFC_ERR_SHAPE, "top2_gating: unknown policy %d", policy);
  if (groups == 0) return MTFC_OK;
  if (groups > INT32_MAX) return fail(MTFC_ERR_SHAPE, "top2_gating: too many groups");
  GateArgs a;
  a.logits = logits; a.parts = parts; a.group_size = group_size; a.experts = experts;
  a.capacity = capacity; a.policy = policy; a.threshold = threshold; a.noise = noise;
  a.idx1 = idx1; a.idx2 = idx2; a.pos1 = pos1; a.pos2 = pos2; a.gate1 = gate1; a.gate2 = gate2;
  a.raw_gates = raw_gates; a.loss_per_group = loss_per_group;
  const int threads = gate_threads(experts, group_size);
  const size_t smem = gate_smem_bytes(experts, threads);
  if (smem > 48 * 1024) {
    static bool attr_set[64] = {false};
    int dev = 0;
    MTFC_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && !attr_set[dev]) {
      MTFC_CUDA(cudaFuncSetAttribute(top2_gating_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      attr_set[dev] = true;
    }
  }
  top2_gating_kernel<<<(unsigned)groups, threads, smem, static_cast<cudaStream_t>(stream)>>>(a);
  MTFC_LAUNCH_CHECK("top2_gating_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_moe_slot_table(const int32_t* idx1, const int32_t* idx2, const int32_t* pos1,
                        const int32_t* pos2, const float* gate1, const float* gate2,
                        int64_t groups, int32_t group_size, int32_t experts, int32_t capacity,
                        int32_t round_gates_to_bf16, int32_t* table, void* stream) {
  if (!idx1 || !idx2 || !pos1 || !pos2 || !gate1 || !gate2 || !table)
    return fail(MTFC_ERR_SHAPE, "slot_table: null argument");
  if (groups < 0 || group_size < 1 || experts < 1 || capacity < 1)
    return fail(MTFC_ERR_SHAPE, "slot_table: bad extents");
  if (groups > INT32_MAX || (long long)experts * capacity > INT32_MAX)
    return fail(MTFC_ERR_SHAPE, "slot_table: extents too large");
  const size_t table_bytes = (size_t)experts * capacity * sizeof(int);
  const int in_smem = table_bytes <= 48 * 1024;
  if (groups == 0) return MTFC_OK;
  slot_table_kernel<<<(unsigned)groups, 256, in_smem ? table_bytes : 0,
                      static_cast<cudaStream_t>(stream)>>>(
      idx1, idx2, pos1, pos2, gate1, gate2, group_size, experts, capacity, round_gates_to_bf16,
      in_smem, table);
  MTFC_LAUNCH_CHECK("slot_table_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_moe_dispatch(const void* x, const int32_t* table, void* out, int64_t outer,
                      int64_t groups_per_outer, int32_t group_size, int32_t experts,
                      int32_t capacity, int64_t row_bytes, void* stream) {
  if (!x || !table || !out) return fail(MTFC_ERR_SHAPE, "dispatch: null argument");
  if (row_bytes < 16 || row_bytes % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "dispatch: row of %lld bytes is not a multiple of 16", (long long)row_bytes);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "dispatch: buffers must be 16-byte aligned");
  if (outer < 0 || groups_per_outer < 0 || group_size < 1 || experts < 1 || capacity < 1)
    return fail(MTFC_ERR_SHAPE, "dispatch: bad extents");
  const long long groups = outer * groups_per_outer;
  const long long rows = groups * experts * capacity;
  if (rows == 0) return MTFC_OK;
  dispatch_rows_kernel<<<grid_for(rows * 32, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), table, static_cast<uint4*>(out), groups, group_size, experts,
      capacity, (int)(row_bytes / 16), groups_per_outer);
  MTFC_LAUNCH_CHECK("dispatch_rows_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_moe_combine(const void* y, int dtype, const int32_t* idx1, const int32_t* idx2,
                     const int32_t* pos1, const int32_t* pos2, const float* gate1,
                     const float* gate2, void* out, int64_t outer, int64_t groups_per_outer,
                     int32_t group_size, int32_t experts, int32_t capacity, int64_t row_elems,
                     void* stream) {
  if (!y || !idx1 || !idx2 || !pos1 || !pos2 || !gate1 || !gate2 || !out)
    return fail(MTFC_ERR_SHAPE, "combine: null argument");
  const long long esz = dtype == MTFC_BF16 ? 2 : 4;
  if (dtype != MTFC_BF16 && dtype != MTFC_F32)
    return fail(MTFC_ERR_UNSUPPORTED, "combine: dtype %d", dtype);
  if ((row_elems * esz) % 16 != 0 || row_elems < 1)
    return fail(MTFC_ERR_SHAPE, "combine: row of %lld elements is not a multiple of 16 bytes", (long long)row_elems);
  if ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "combine: buffers must be 16-byte aligned");
  const long long groups = outer * groups_per_outer;
  const long long tokens = groups * group_size;
  if (tokens == 0) return MTFC_OK;
  const int vec = (int)(row_elems * esz / 16);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == MTFC_BF16)
    combine_rows_bf16_kernel<<<grid_for(tokens * 32, 256), 256, 0, s>>>(
        static_cast<const uint4*>(y), idx1, idx2, pos1, pos2, gate1, gate2,
        static_cast<uint4*>(out), groups, group_size, experts, capacity, vec, groups_per_outer);
  else
    combine_rows_f32_kernel<<<grid_for(tokens * 32, 256), 256, 0, s>>>(
        static_cast<const float4*>(y), idx1, idx2, pos1, pos2, gate1, gate2,
        static_cast<float4*>(out), groups, group_size, experts, capacity, vec, groups_per_outer);
  MTFC_LAUNCH_CHECK("combine_rows_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_moe_dispatch_weighted(const void* x, int dtype, const int32_t* table, const int32_t* idx1,
                               const int32_t* pos1, const float* gate1, const float* gate2,
                               void* out, int64_t outer, int64_t groups_per_outer,
                               int32_t group_size, int32_t experts, int32_t capacity,
                               int64_t row_elems, void* stream) {
  if (!x || !table || !idx1 || !pos1 || !gate1 || !gate2 || !out)
    return fail(MTFC_ERR_SHAPE, "dispatch_weighted: null argument");
  if (dtype != MTFC_BF16 && dtype != MTFC_F32)
    return fail(MTFC_ERR_UNSUPPORTED, "dispatch_weighted: dtype %d", dtype);
  if (outer < 0 || groups_per_outer < 0 || group_size < 1 || experts < 1 || capacity < 1)
    return fail(MTFC_ERR_SHAPE, "dispatch_weighted: bad extents");
  const long long esz = dtype == MTFC_BF16 ? 2 : 4;
  if (row_elems < 1 || (row_elems * esz) % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "dispatch_weighted: row of %lld elements is not a multiple of 16 bytes",
                (long long)row_elems);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "dispatch_weighted: buffers must be 16-byte aligned");
  const long long groups = outer * groups_per_outer;
  const long long rows = groups * experts * capacity;
  if (rows == 0) return MTFC_OK;
  const int vec = (int)(row_elems * esz / 16);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == MTFC_BF16)
    dispatch_rows_weighted_kernel<true><<<grid_for(rows * 32, 256), 256, 0, s>>>(
        static_cast<const uint4*>(x), table, idx1, pos1, gate1, gate2, static_cast<uint4*>(out),
        groups, group_size, experts, capacity, vec, groups_per_outer);
  else
    dispatch_rows_weighted_kernel<false><<<grid_for(rows * 32, 256), 256, 0, s>>>(
        static_cast<const uint4*>(x), table, idx1, pos1, gate1, gate2, static_cast<uint4*>(out),
        groups, group_size, experts, capacity, vec, groups_per_outer);
  MTFC_LAUNCH_CHECK("dispatch_rows_weighted_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_moe_combine_gate_grad(const void* y, const void* dout, int dtype, const int32_t* idx1,
                               const int32_t* idx2, const int32_t* pos1, const int32_t* pos2,
                               const float* gate1, const float* gate2, float* dgate1,
                               float* dgate2, int64_t outer, int64_t groups_per_outer,
                               int32_t group_size, int32_t experts, int32_t capacity,
                               int64_t row_elems, void* stream) {
  if (!y || !dout || !idx1 || !idx2 || !pos1 || !pos2 || !gate1 || !gate2 || !dgate1 || !dgate2)
    return fail(MTFC_ERR_SHAPE, "combine_gate_grad: null argument");
  if (dtype != MTFC_BF16 && dtype != MTFC_F32)
    return fail(MTFC_ERR_UNSUPPORTED, "combine_gate_grad: dtype %d", dtype);
  if (outer < 0 || groups_per_outer < 0 || group_size < 1 || experts < 1 || capacity < 1)
    return fail(MTFC_ERR_SHAPE, "combine_gate_grad: bad extents");
  const long long esz = dtype == MTFC_BF16 ? 2 : 4;
  if (row_elems < 1 || (row_elems * esz) % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "combine_gate_grad: row of %lld elements is not a multiple of 16 bytes",
                (long long)row_elems);
  if ((reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(dout)) % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "combine_gate_grad: buffers must be 16-byte aligned");
  const long long groups = outer * groups_per_outer;
  const long long tokens = groups * group_size;
  if (tokens == 0) return MTFC_OK;
  const int vec = (int)(row_elems * esz / 16);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == MTFC_BF16)
    combine_gate_grad_kernel<true><<<grid_for(tokens * 32, 256), 256, 0, s>>>(
        static_cast<const uint4*>(y), static_cast<const uint4*>(dout), idx1, idx2, pos1, pos2, gate1,
        gate2, dgate1, dgate2, groups, group_size, experts, capacity, vec, groups_per_outer);
  else
    combine_gate_grad_kernel<false><<<grid_for(tokens * 32, 256), 256, 0, s>>>(
        static_cast<const uint4*>(y), static_cast<const uint4*>(dout), idx1, idx2, pos1, pos2, gate1,
        gate2, dgate1, dgate2, groups, group_size, experts, capacity, vec, groups_per_outer);
  MTFC_LAUNCH_CHECK("combine_gate_grad_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_moe_dispatch_noalloc(const void* x, const int32_t* idx1, const int32_t* idx2,
                              const int32_t* pos1, const int32_t* pos2, const float* gate1,
                              const float* gate2, void* out, int64_t outer,
                              int64_t groups_per_outer, int32_t group_size, int32_t experts,
                              int32_t capacity, int64_t row_bytes, int32_t round_gates_to_bf16,
                              void* stream) {
  if (!x || !idx1 || !idx2 || !pos1 || !pos2 || !gate1 || !gate2 || !out)
    return fail(MTFC_ERR_SHAPE, "dispatch_noalloc: null argument");
  if (outer < 0 || groups_per_outer < 0 || group_size < 1 || experts < 1 || capacity < 1)
    return fail(MTFC_ERR_SHAPE, "dispatch_noalloc: bad extents");
  if (row_bytes < 16 || row_bytes % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "dispatch_noalloc: row of %lld bytes is not a multiple of 16",
                (long long)row_bytes);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "dispatch_noalloc: buffers must be 16-byte aligned");
  const long long groups = outer * groups_per_outer;
  const long long entries = groups * experts * capacity;
  if (entries > kNoAllocSlotCapacity)
    return fail(MTFC_ERR_SHAPE,
                "dispatch_noalloc: groups*experts*capacity = %lld exceeds the built-in scratch of "
                "%lld entries; use mtfc_moe_slot_table + mtfc_moe_dispatch with your own table",
                entries, kNoAllocSlotCapacity);
  if ((size_t)experts * capacity * sizeof(int) > 48 * 1024)
    return fail(MTFC_ERR_SHAPE, "dispatch_noalloc: experts*capacity=%d too large", experts * capacity);
  if (entries == 0) return MTFC_OK;
  int* table = nullptr;
  int rc = noalloc_slot_table_ptr(&table);
  if (rc != MTFC_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The table is rewritten in full for the entries this call uses, so nothing
  // left over from an earlier call is ever read.
  slot_table_kernel<<<(unsigned)groups, 256, (size_t)experts * capacity * sizeof(int), s>>>(
      idx1, idx2, pos1, pos2, gate1, gate2, group_size, experts, capacity, round_gates_to_bf16,
      1, table);
  MTFC_LAUNCH_CHECK("slot_table_kernel");
  dispatch_rows_kernel<<<grid_for(entries * 32, 256), 256, 0, s>>>(
      static_cast<const uint4*>(x), table, static_cast<uint4*>(out), groups, group_size, experts,
      capacity, (int)(row_bytes / 16), groups_per_outer);
  MTFC_LAUNCH_CHECK("dispatch_rows_kernel");
  count_launch(2);
  return MTFC_OK;
}

}  // extern "C"
