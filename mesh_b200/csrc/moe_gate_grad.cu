// Backward of the top-2 (and top-1 "switch") gating as one kernel: from the gate
// logits, the routing decisions and the gradients of (gate_1, gate_2, loss) to
// the gradient of the logits.
//
// The reference differentiates its op chain (transformer/moe.py:1384-1424,
// 1485-1494): softmax, the two picked gates (top_1's gradient is a one-hot
// scatter, ops.py:4916-4920), their renormalisation g_k = b_k / (b_1 + b_2 +
// 1e-9) times the capacity / policy masks (comparisons: constants), and the
// load-balancing loss mean_{g,e}(mean_s raw · density_1) · E², in which the
// fraction density_1 of positions choosing an expert is a constant as well.
// That is some sixty element-wise and reduce operations on [tokens, E] tensors;
// here a thread owns a token:
//
//   raw      = softmax(logits)                    (max, exp, sum: fp32)
//   d raw[e] = dloss · E / (G_total · S) · density_1[g, e]
//   d raw[i1] += dg1·k1·(1/den − b1/den²) − dg2·k2·b2/den²
//   d raw[i2] += dg2·k2·(1/den − b2/den²) − dg1·k1·b1/den²      (top-1: d raw[i1] += dg1·k1)
//   d logits = raw ⊙ (d raw − <raw, d raw>)
//
// One CTA per group: it first counts the group's first choices per expert in
// shared memory (density_1), then walks the group's tokens.  The two products
// that follow (d inputs = d logits · Wᵀ, d W = inputsᵀ · d logits) are ordinary
// einsums.

#include "common.cuh"

namespace mtfc {
namespace {

constexpr int kGradMaxExperts = 64;

struct GateGradArgs {
  const float* logits;   // [groups, S, E]
  const int* idx1;
  const int* idx2;
  const float* gate1;    // gates as the forward pass returned them: 0 where dropped
  const float* gate2;
  const float* dgate1;   // may be null: no gradient arrives
  const float* dgate2;
  const float* dloss;    // device scalar, may be null
  float* dlogits;
  int group_size, experts;
  float loss_scale;      // E / (G_total * S)
  int top1_only;
};

template <int EP>
__global__ void __launch_bounds__(256)
moe_gate_grad_kernel(const GateGradArgs a) {
  __shared__ int count[EP];
  const int g = blockIdx.x, S = a.group_size, E = a.experts;
  const long long tok0 = (long long)g * S;
  for (int e = threadIdx.x; e < EP; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int s = threadIdx.x; s < S; s += blockDim.x) {
    const int i1 = a.idx1[tok0 + s];
    if (i1 >= 0 && i1 < E) atomicAdd(&count[i1], 1);
  }
  __syncthreads();
  const float dloss = a.dloss ? *a.dloss : 0.f;
  const float from_loss = dloss * a.loss_scale / (float)S;   // times count = density * S
  for (int s = threadIdx.x; s < S; s += blockDim.x) {
    const long long t = tok0 + s;
    const float* row = a.logits + t * E;
    float r[EP];
    float mx = -3.0e38f;
#pragma unroll
    for (int e = 0; e < EP; ++e) {
      r[e] = e < E ? row[e] : -3.0e38f;
      mx = fmaxf(mx, r[e]);
    }
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < EP; ++e)
      if (e < E) sum += expf(r[e] - mx);
    const float lse = logf(sum) + mx;
    const int i1 = a.idx1[t], i2 = a.idx2[t];
    float b1 = 0.f, b2 = 0.f;
#pragma unroll
    for (int e = 0; e < EP; ++e) {
      r[e] = e < E ? expf(r[e] - lse) : 0.f;
      if (e == i1) b1 = r[e];
      if (e == i2) b2 = r[e];
    }
    const float k1 = a.gate1[t] != 0.f ? 1.f : 0.f;
    const float k2 = a.gate2[t] != 0.f ? 1.f : 0.f;
    const float d1 = (a.dgate1 ? a.dgate1[t] : 0.f) * k1;
    const float d2 = (a.dgate2 ? a.dgate2[t] : 0.f) * k2;
    float at1, at2;
    if (a.top1_only) {
      at1 = d1;
      at2 = 0.f;
    } else {
      const float den = b1 + b2 + 1e-9f;
      const float inv = 1.0f / den, inv2 = inv * inv;
      at1 = d1 * (inv - b1 * inv2) - d2 * b2 * inv2;
      at2 = d2 * (inv - b2 * inv2) - d1 * b1 * inv2;
    }
    float dot = 0.f;
    float dr[EP];
#pragma unroll
    for (int e = 0; e < EP; ++e) {
      float d = e < E ? from_loss * (float)count[e] : 0.f;
      if (e == i1) d += at1;
      if (e == i2) d += at2;
      dr[e] = d;
      dot += r[e] * d;
    }
    float* out = a.dlogits + t * E;
#pragma unroll
    for (int e = 0; e < EP; ++e)
      if (e < E) out[e] = r[e] * (dr[e] - dot);
  }
}

}  // namespace
}  // namespace mtfc

using namespace mtfc;

extern "C" {

int mtfc_moe_gate_grad(const float* logits, const int32_t* idx1, const int32_t* idx2,
                       const float* gate1, const float* gate2, const float* dgate1,
                       const float* dgate2, const float* dloss, int64_t groups, int32_t group_size,
                       int32_t experts, int64_t num_groups_total, int32_t top1_only, float* dlogits,
                       void* stream) {
  if (!logits || !idx1 || !idx2 || !gate1 || !gate2 || !dlogits)
    return fail(MTFC_ERR_SHAPE, "gate_grad: null argument");
  if (groups < 0 || group_size < 1 || experts < 1 || num_groups_total < 1 || groups > INT32_MAX)
    return fail(MTFC_ERR_SHAPE, "gate_grad: bad extents");
  if (experts > kGradMaxExperts)
    return fail(MTFC_ERR_UNSUPPORTED, "gate_grad: at most %d experts (got %d)", kGradMaxExperts, experts);
  if (groups == 0) return MTFC_OK;
  GateGradArgs a;
  a.logits = logits; a.idx1 = idx1; a.idx2 = idx2; a.gate1 = gate1; a.gate2 = gate2;
  a.dgate1 = dgate1; a.dgate2 = dgate2; a.dloss = dloss; a.dlogits = dlogits;
  a.group_size = group_size; a.experts = experts;
  a.loss_scale = (float)experts / ((float)num_groups_total * (float)group_size);
  a.top1_only = top1_only;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)groups;
  if (experts <= 16) moe_gate_grad_kernel<16><<<grid, 256, 0, s>>>(a);
  else if (experts <= 32) moe_gate_grad_kernel<32><<<grid, 256, 0, s>>>(a);
  else moe_gate_grad_kernel<64><<<grid, 256, 0, s>>>(a);
  MTFC_LAUNCH_CHECK("moe_gate_grad_kernel");
  count_launch(1);
  return MTFC_OK;
}

}  // extern "C"
