// K2/K3, single pass over the activations: gate logits, softmax, top-2 and
// renormalised gates in one tcgen05 kernel, then positions / capacity in a
// small per-group scan kernel.
//
// Replaces, for bf16 activations, the sequence "gate-logit GEMM -> logits in
// HBM -> top2_gating_kernel" for `_top_2_gating`
// (mesh_tensorflow/transformer/moe.py:1380-1513): the activations are read
// once (2 bytes x d_model per token), nothing but 16 bytes of routing per
// token is written, and the softmax / top-2 arithmetic runs with one thread
// per token on values held in registers.
//
//   gate_top2_fused   persistent, one CTA per SM, 192 threads:
//       warp 0     TMA producer: x tile (128 tokens x 64) + gate-kernel tile
//                  (3*EP rows x 64) per K block into a ring of swizzled stages
//       warp 1     tcgen05.mma 128 x 3EP x 16 into one of two TMEM accumulators
//       warps 2-5  epilogue: thread i owns token row i of the tile: reads the
//                  3*EP accumulator columns (hi | mid | lo parts of the fp32
//                  gate kernel, so the bf16 products add up to fp32 accuracy),
//                  frees the accumulator, then softmax in the exp(x - logsumexp)
//                  form, top-1, masked top-2 (ties: lowest index), gates
//                  renormalised with reciprocal-then-multiply.  Column sums of
//                  the raw gates (for the load-balancing loss) leave the CTA as
//                  one partial row per tile, added in a fixed order.
//       Tiles never straddle a group: tile (g, c) covers tokens [128c, 128c+128)
//       of group g and ignores rows past the group's end.
//   top2_positions    one CTA per group: position-in-expert of both choices by
//                  warp match/popc ranks plus a cross-warp scan, second-expert
//                  policy, capacity masks, loss; optionally the (expert, slot)
//                  -> token table the dispatch kernel reads.
//
// Every mbarrier wait is bounded (tcgen05_ptx.cuh); on expiry the kernel raises
// the status word, frees its TMEM and returns.

#include "tcgen05_ptx.cuh"

namespace mtfc {
namespace {

constexpr int TILE_TOKENS = 128;
constexpr int GBK = 64;  // bf16 per K block = one 128-byte swizzle row
constexpr int G_UMMA_K = 16;
constexpr int X_STAGE_BYTES = TILE_TOKENS * GBK * 2;  // 16 KiB
constexpr int MAX_STAGES = 8;
constexpr int G_THREADS = 192;
constexpr int G_EPI_WARPS = 4;
constexpr int G_TMEM_COLS = 512;
constexpr int G_ACC_STRIDE = 256;  // TMEM columns between the two accumulators
constexpr int kMaxGateExperts = 64;

struct GateFusedArgs {
  int group_size, experts, m;
  int renormalize;  // 0: gate_1 is the raw top-1 gate and gate_2 is 0 (top-1 routing)
  int tile_rows;  // tokens per tile: 128, or 64 when that fills the SMs more evenly
  int tiles_per_group;
  int big_per_group;  // tiles_per_group / R rounded up: passes a CTA makes over a group
  long long num_tiles;
  int stages;
  int* idx1;
  int* idx2;
  float* gate1;
  float* gate2;
  float* raw_gates;  // [tokens, experts] or null
  float* tile_sums;  // [num_tiles, EP]: column sums of the raw gates per tile
  int* tile_counts;  // [num_tiles, 2, EP]: tokens of the tile choosing each expert 1st / 2nd
  int* rank1;        // per token: tokens of its tile before it with the same first choice
  int* rank2;        // the same for the second choice among tokens that pass the policy; -1 if not
  int policy;
  float threshold;
  const float* noise;
  unsigned* groups_done;  // counter the positions kernel's CTAs take tickets from; zeroed here
  int* status;
};

__device__ __forceinline__ void tc_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void epi_warps_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(32 * G_EPI_WARPS) : "memory");
}

// Programmatic dependent launch: the three kernels of one gating call follow one
// another closely and each is short, so the next one is allowed onto the SMs while
// its predecessor still runs (launch_dependents) and does its set-up there; it
// touches global memory only after griddepcontrol.wait, which returns when the
// predecessor grid has completed and its writes are visible.  Both instructions do
// nothing in a kernel that was launched without the attribute.
__device__ __forceinline__ void let_next_kernel_start() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void wait_for_previous_kernel() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// fp32 gate kernel [m, E] -> bf16 [3*EP, m]: row p*EP + e holds part p (hi, mid,
// lo) of column e; rows of experts in [E, EP) are zero.
__global__ void split_gate_weights_kmajor_kernel(const float* __restrict__ w, long long m, int e,
                                                 int ep, __nv_bfloat16* __restrict__ out) {
  let_next_kernel_start();
  const long long n = m * ep;
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += step) {
    const int col = (int)(i / m);        // expert (padded)
    const long long row = i - col * m;   // d_model index: consecutive threads, consecutive rows
    __nv_bfloat16 hi = __float2bfloat16_rn(0.f), mid = hi, lo = hi;
    if (col < e) {
      const float v = w[row * e + col];
      hi = __float2bfloat16_rn(v);
      const float r1 = v - __bfloat162float(hi);
      mid = __float2bfloat16_rn(r1);
      const float r2 = r1 - __bfloat162float(mid);
      lo = __float2bfloat16_rn(r2);
    }
    out[(long long)col * m + row] = hi;
    out[(long long)(ep + col) * m + row] = mid;
    out[(long long)(2 * ep + col) * m + row] = lo;
  }
}

// R tiles of 128 tokens per pass share every K block of the gate kernel in shared
// memory (R = 2 needs 3 * EP <= 128 accumulator columns per tile).
template <int EP, int R>
__global__ void __launch_bounds__(G_THREADS, 1)
gate_top2_fused(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                const GateFusedArgs a) {
  constexpr int N = 3 * EP;
  constexpr int W_STAGE_BYTES = N * GBK * 2;
  constexpr int XS_BYTES = R * X_STAGE_BYTES;   // activations per stage
  static_assert(R == 1 || 3 * EP <= 128, "two tiles per pass need 3*EP <= 128 accumulator columns");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  const int ST = a.stages;
  const uint32_t off_w = (uint32_t)ST * XS_BYTES;
  const uint32_t off_sums = off_w + (uint32_t)ST * W_STAGE_BYTES;
  const uint32_t off_cnt = off_sums + 2 * G_EPI_WARPS * EP * 4;
  const uint32_t off_bar = off_cnt + 2 * 2 * G_EPI_WARPS * EP * 4;
  const uint32_t off_misc = off_bar + (2 * MAX_STAGES + 4) * 8;
  const uint32_t bar_base = smem_base + off_bar;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
  auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * MAX_STAGES + b); };
  auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * MAX_STAGES + 2 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + off_misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + off_misc + 4);
  float* warp_sums = reinterpret_cast<float*>(smem + off_sums);  // [2][G_EPI_WARPS][EP]
  int* warp_cnt = reinterpret_cast<int*>(smem + off_cnt);        // [2][2 choices][G_EPI_WARPS][EP]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tmem_full_bar(b), 1);
      mbar_init(tmem_empty_bar(b), G_EPI_WARPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_base + off_misc),
                 "r"(G_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_kb = (a.m + GBK - 1) / GBK;
  // barriers, TMEM and descriptors are in place: from here on global memory is touched
  wait_for_previous_kernel();
  let_next_kernel_start();
  if (blockIdx.x == 0 && threadIdx.x == 0) *a.groups_done = 0u;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < a.num_tiles && ok; t += gridDim.x) {
        const long long g = t / a.big_per_group;
        const int c = (int)(t - g * a.big_per_group) * R;
        const long long row0 = g * a.group_size + (long long)c * a.tile_rows;
        // with 64-token tiles the box is half a stage: rows 64..127 of the stage keep
        // whatever they held, and the accumulator rows they produce are never read
        const uint32_t x_bytes = (uint32_t)a.tile_rows * GBK * 2;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), R * x_bytes + W_STAGE_BYTES);
#pragma unroll
          for (int h = 0; h < R; ++h)   // a second tile past the group's end is loaded and ignored
            tma_load_3d(smem_base + stage * XS_BYTES + h * X_STAGE_BYTES, &map_x, full_bar(stage),
                        kb * GBK, (int)(row0 + (long long)h * a.tile_rows), 0);
          tma_load_3d(smem_base + off_w + stage * W_STAGE_BYTES, &map_w, full_bar(stage), kb * GBK,
                      0, 0);
          if (++stage == ST) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok && a.status) atomicExch(a.status, MTFC_ERR_TIMEOUT);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // kind::f16 instruction descriptor: fp32 accumulator, bf16 operands, both K-major
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) |
                             ((uint32_t)(TILE_TOKENS >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long local = 0;
      for (long long t = blockIdx.x; t < a.num_tiles && ok; t += gridDim.x, ++local) {
        const int buf = (int)(local & 1);
        const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
        if (!mbar_wait(tmem_empty_bar(buf), acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * G_ACC_STRIDE);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sx = smem_base + stage * XS_BYTES;
          const uint32_t sw = smem_base + off_w + stage * W_STAGE_BYTES;
#pragma unroll
          for (int ks = 0; ks < GBK / G_UMMA_K; ++ks) {
            const uint64_t db = make_smem_desc(sw + ks * G_UMMA_K * 2, 16, 1024);
#pragma unroll
            for (int h = 0; h < R; ++h) {
              const uint64_t da = make_smem_desc(sx + h * X_STAGE_BYTES + ks * G_UMMA_K * 2, 16, 1024);
              tc_mma_bf16(d_tmem + (uint32_t)(h * (G_ACC_STRIDE / 2)), da, db, idesc,
                          (kb | ks) != 0 ? 1u : 0u);
            }
          }
          tc_commit(empty_bar(stage));
          if (++stage == ST) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(tmem_full_bar(buf));
      }
      if (!ok && a.status) atomicExch(a.status, MTFC_ERR_TIMEOUT);
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;   // TMEM lane quarter this warp may read
    const int ew = warp - 2;  // 0..3
    const int E = a.experts;
    bool ok = true;
    long long local = 0;
    for (long long t = blockIdx.x; t < a.num_tiles && ok; t += gridDim.x, ++local) {
      const int buf = (int)(local & 1);
      const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
      const long long g = t / a.big_per_group;
      const int c0 = (int)(t - g * a.big_per_group) * R;
      const int row = q * 32 + lane;
      ok = __all_sync(0xffffffffu, mbar_wait(tmem_full_bar(buf), acc_phase, abort_flag));
      if (!ok) {
        // a warp that gave up still counts at the column-sum barriers of this pass, so
        // that warps which got through the wait are not left standing there
        for (int h = 0; h < R; ++h) asm volatile("bar.arrive 1, %0;" ::"n"(32 * G_EPI_WARPS) : "memory");
        break;
      }
      tc_fence_after();
#pragma unroll 1
      for (int h = 0; h < R; ++h) {
      const int c = c0 + h;                      // tile of the group this half is
      const long long slot = local * R + h;      // picks the double-buffered scratch rows
      const int s_in_group = c * a.tile_rows + row;
      const bool live = row < a.tile_rows && s_in_group < a.group_size;
      const long long tok = g * a.group_size + s_in_group;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) +
                             (uint32_t)(buf * G_ACC_STRIDE + h * (G_ACC_STRIDE / 2));
      float r[EP];
#pragma unroll
      for (int ch = 0; ch < EP / 16; ++ch) {
        uint32_t hi[16], mid[16], lo[16];
        tc_ld_32x16(t_row + ch * 16, hi);
        tc_ld_32x16(t_row + EP + ch * 16, mid);
        tc_ld_32x16(t_row + 2 * EP + ch * 16, lo);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j)
          r[ch * 16 + j] = (__uint_as_float(hi[j]) + __uint_as_float(mid[j])) + __uint_as_float(lo[j]);
      }
      if (h == R - 1) {
        // the accumulators are in registers: hand the buffer back before the arithmetic
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tmem_empty_bar(buf));
      }

      float mx = r[0];
#pragma unroll
      for (int e = 1; e < EP; ++e)
        if (e < E) mx = fmaxf(mx, r[e]);
      float sum = 0.f;
#pragma unroll
      for (int e = 0; e < EP; ++e)
        if (e < E) sum += expf(r[e] - mx);
      const float lse = logf(sum) + mx;
      int i1 = 0, i2 = 0;
      float b1 = -1.f, b2 = -1.f;
#pragma unroll
      for (int e = 0; e < EP; ++e) {
        const float p = e < E ? expf(r[e] - lse) : 0.f;
        r[e] = p;
        if (e < E && p > b1) { b1 = p; i1 = e; }
      }
#pragma unroll
      for (int e = 0; e < EP; ++e) {
        const float p = (e == i1) ? 0.f : r[e];
        if (e < E && p > b2) { b2 = p; i2 = e; }
      }
      const float recip = 1.0f / ((b1 + b2) + 1e-9f);
      const float g1n = a.renormalize ? b1 * recip : b1;
      const float g2n = a.renormalize ? b2 * recip : 0.f;
      // second-expert policy (moe.py:1446-1467), on the renormalised gate
      bool m2 = false;
      if (live) {
        switch (a.policy) {
          case MTFC_MOE_POLICY_ALL: m2 = true; break;
          case MTFC_MOE_POLICY_THRESHOLD: m2 = g2n > a.threshold; break;
          case MTFC_MOE_POLICY_RANDOM:
            m2 = a.noise[tok] < g2n * (1.0f / fmaxf(a.threshold, 1e-9f));
            break;
          default: m2 = false;   // none, switch
        }
      }
      // rank among the tile's earlier tokens with the same choice: inside the warp by
      // match/popc, across the four warps through per-warp counts (added after the barrier)
      int* cnt_a = warp_cnt + (((slot & 1) * 2 + 0) * G_EPI_WARPS + ew) * EP;
      int* cnt_b = warp_cnt + (((slot & 1) * 2 + 1) * G_EPI_WARPS + ew) * EP;
      for (int e = lane; e < EP; e += 32) { cnt_a[e] = 0; cnt_b[e] = 0; }
      __syncwarp();
      const unsigned lt_mask = (1u << lane) - 1u;
      const unsigned same1 = __match_any_sync(0xffffffffu, live ? i1 : -1 - lane);
      int rank1 = __popc(same1 & lt_mask);
      if (live && rank1 == 0) cnt_a[i1] = __popc(same1);
      const unsigned same2 = __match_any_sync(0xffffffffu, m2 ? i2 : -1 - lane);
      int rank2 = __popc(same2 & lt_mask);
      if (m2 && rank2 == 0) cnt_b[i2] = __popc(same2);
      if (live) {
        a.idx1[tok] = i1;
        a.idx2[tok] = i2;
        a.gate1[tok] = g1n;
        a.gate2[tok] = g2n;
        if (a.raw_gates) {
          float* dst = a.raw_gates + tok * E;
#pragma unroll
          for (int e = 0; e < EP; ++e)
            if (e < E) dst[e] = r[e];
        }
      } else {
#pragma unroll
        for (int e = 0; e < EP; ++e) r[e] = 0.f;   // rows past the group's end add nothing
      }
      // column sums over the warp's 32 rows: reduce-scatter over the lanes (a
      // fixed tree), after which lane l holds the sums of EP/32 (or, for EP = 16,
      // half a) column
#pragma unroll
      for (int k = 0; k < 5; ++k) {
        const int off = 16 >> k;
        const int before = (EP >> k) > 1 ? (EP >> k) : 1;   // values per lane entering the step
        if (before > 1) {
          const int half = before >> 1;
          const bool upper = (lane & off) != 0;
#pragma unroll
          for (int i = 0; i < EP / 2; ++i) {
            if (i < half) {
              const float send = upper ? r[i] : r[i + half];
              const float keep = upper ? r[i + half] : r[i];
              r[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
            }
          }
        } else {
          r[0] += __shfl_xor_sync(0xffffffffu, r[0], off);
        }
      }
      float* mine = warp_sums + ((slot & 1) * G_EPI_WARPS + ew) * EP;
      if (EP >= 32) {
#pragma unroll
        for (int i = 0; i < EP / 32; ++i) mine[lane * (EP / 32) + i] = r[i];
      } else if ((lane & 1) == 0) {
        mine[lane >> 1] = r[0];
      }
      epi_warps_sync();
      {
        // warps earlier in token order: lane quarter q' < q sits in epilogue warp (q' + 2) & 3
        const int* all_a = warp_cnt + ((slot & 1) * 2 + 0) * G_EPI_WARPS * EP;
        const int* all_b = warp_cnt + ((slot & 1) * 2 + 1) * G_EPI_WARPS * EP;
        for (int qq = 0; qq < q; ++qq) {
          const int w = (qq + 2) & 3;
          if (live) rank1 += all_a[w * EP + i1];
          if (m2) rank2 += all_b[w * EP + i2];
        }
        if (live) {
          a.rank1[tok] = rank1;
          a.rank2[tok] = m2 ? rank2 : -1;
        }
      }
      const int tid = ew * 32 + lane;
      if (tid < EP && c < a.tiles_per_group) {   // a half past the group's end has no slot
        const long long tile = g * a.tiles_per_group + c;
        const float* ws = warp_sums + (slot & 1) * G_EPI_WARPS * EP;
        // rows in token order: warps 2..5 hold lane quarters 2, 3, 0, 1
        const float s = ((ws[2 * EP + tid] + ws[3 * EP + tid]) + ws[0 * EP + tid]) + ws[1 * EP + tid];
        a.tile_sums[tile * EP + tid] = s;
        const int* ca = warp_cnt + ((slot & 1) * 2 + 0) * G_EPI_WARPS * EP + tid;
        const int* cb = warp_cnt + ((slot & 1) * 2 + 1) * G_EPI_WARPS * EP + tid;
        a.tile_counts[(tile * 2 + 0) * EP + tid] = ca[0] + ca[EP] + ca[2 * EP] + ca[3 * EP];
        a.tile_counts[(tile * 2 + 1) * EP + tid] = cb[0] + cb[EP] + cb[2 * EP] + cb[3 * EP];
      }
      }   // halves
    }
    if (!ok && lane == 0 && a.status) atomicExch(a.status, MTFC_ERR_TIMEOUT);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(G_TMEM_COLS)
                 : "memory");
  }
}

__device__ __forceinline__ bool gate_nonzero_bf16(float g) {
  return __bfloat162float(__float2bfloat16_rn(g)) != 0.0f;
}

struct PositionArgs {
  int group_size, experts, capacity;
  const int* idx1;
  const int* idx2;
  int* pos1;     // in: rank inside the tile; out: position in the expert's buffer
  int* pos2;     // in: rank inside the tile among policy-passing tokens, -1 if none; out: position
  float* gate1;  // in: renormalised gates; out: zeroed where dropped
  float* gate2;
  const float* tile_sums;   // [groups, tiles_per_group, ep]
  const int* tile_counts;   // [groups, tiles_per_group, 2, ep]
  int tiles_per_group, tile_rows, ep;
  float* loss_per_group;
  float* loss_mean;        // sum over groups / num_groups_total, or null
  float inv_groups_total;
  unsigned* groups_done;
  int* table;  // [groups, experts, capacity] or null
  int table_in_smem;
  int round_bf16;
};

// One CTA per group.  The fused kernel left, per token, its rank among the
// earlier tokens of its tile with the same choice and, per tile, the number of
// tokens choosing each expert; an exclusive scan of those counts over the
// group's tiles (one thread per expert) gives every tile's base, and
// position = base + rank.  Second choices start after the kept first choices
// (moe.py:1488-1490).  Shared memory: base1[tiles][E], base2[tiles][E], tot1[E],
// sums[tiles][E], slots[E*C] (if a table is built there).
__global__ void __launch_bounds__(1024)
top2_positions_kernel(PositionArgs a) {
  extern __shared__ int ismem[];
  const int E = a.experts, S = a.group_size, C = a.capacity;
  const int T = blockDim.x, K = a.tiles_per_group;
  int* base1 = ismem;
  int* base2 = base1 + K * E;
  int* tot1 = base2 + K * E;
  float* sums = reinterpret_cast<float*>(tot1 + E);   // [K][E]
  const int g = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long tok0 = (long long)g * S;
  // the group's slot table is built in shared memory when it fits there, else in place
  int* slots = a.table_in_smem ? reinterpret_cast<int*>(sums + K * E) : a.table + (long long)g * E * C;
  wait_for_previous_kernel();

  // this thread's first token, requested now so that it arrives while the scans run
  int i1_first = 0, i2_first = 0, r1_first = 0, r2_first = -1;
  float g1_first = 0.f, g2_first = 0.f;
  if (tid < S) {
    i1_first = a.idx1[tok0 + tid];
    i2_first = a.idx2[tok0 + tid];
    r1_first = a.pos1[tok0 + tid];
    r2_first = a.pos2[tok0 + tid];
    g1_first = a.gate1[tok0 + tid];
    g2_first = a.gate2[tok0 + tid];
  }
  // every tile's counts and column sums in one round of loads, then the scans run
  // out of shared memory
  for (int i = tid; i < K * E; i += T) {
    const int k = i / E, e = i - k * E;
    const long long tile = (long long)g * K + k;
    base1[i] = a.tile_counts[(tile * 2 + 0) * a.ep + e];
    base2[i] = a.tile_counts[(tile * 2 + 1) * a.ep + e];
    sums[i] = a.tile_sums[tile * a.ep + e];
  }
  if (a.table)
    for (int i = tid; i < E * C; i += T) slots[i] = -1;
  __syncthreads();
  for (int e = tid; e < E; e += T) {
    int run = 0;
    for (int k = 0; k < K; ++k) {
      const int n = base1[k * E + e];
      base1[k * E + e] = run;
      run += n;
    }
    tot1[e] = run;
    int run2 = min(run, C);   // second choices queue behind the kept first choices
    for (int k = 0; k < K; ++k) {
      const int n = base2[k * E + e];
      base2[k * E + e] = run2;
      run2 += n;
    }
    float proxy = 0.f;
    for (int k = 0; k < K; ++k) proxy += sums[k * E + e];
    sums[e] = proxy;   // row 0 now holds the group's column sums
  }
  __syncthreads();

  if (warp == 0) {   // load-balancing loss on the pre-capacity counts (moe.py:1420-1424)
    float part = 0.f;
    const float inv_s = 1.0f / (float)S;
    for (int e = lane; e < E; e += 32) part += (sums[e] * inv_s) * ((float)tot1[e] * inv_s);
    for (int s = 16; s > 0; s >>= 1) part += __shfl_xor_sync(0xffffffffu, part, s);
    if (lane == 0) a.loss_per_group[g] = part * (1.0f / (float)E) * (float)(E * E);
  }

  for (int s = tid; s < S; s += T) {
    const long long t = tok0 + s;
    const int k = s / a.tile_rows;
    // the first round's token was fetched before the scans
    const bool pre = s == tid;
    const int i1 = pre ? i1_first : a.idx1[t], i2 = pre ? i2_first : a.idx2[t];
    const int r1 = pre ? r1_first : a.pos1[t], r2 = pre ? r2_first : a.pos2[t];
    const bool m2 = r2 >= 0;
    const int p1 = base1[k * E + i1] + r1;
    const int p2 = m2 ? base2[k * E + i2] + r2 : 0;
    const bool keep1 = p1 < C;
    const bool keep2 = m2 && p2 < C;
    const float g1 = keep1 ? (pre ? g1_first : a.gate1[t]) : 0.f;
    const float g2 = keep2 ? (pre ? g2_first : a.gate2[t]) : 0.f;
    a.pos1[t] = p1;
    a.pos2[t] = p2;
    a.gate1[t] = g1;
    a.gate2[t] = g2;
    if (a.table) {
      if (keep1 && (a.round_bf16 ? gate_nonzero_bf16(g1) : g1 != 0.f)) slots[i1 * C + p1] = s;
      if (keep2 && (a.round_bf16 ? gate_nonzero_bf16(g2) : g2 != 0.f)) slots[i2 * C + p2] = s;
    }
  }
  if (a.table && a.table_in_smem) {
    __syncthreads();
    for (int i = tid; i < E * C; i += T) a.table[(long long)g * E * C + i] = slots[i];
  }
  // the CTA that finishes last adds the per-group losses, always in the same order
  if (a.loss_mean && warp == 0) {
    unsigned ticket = 0;
    if (lane == 0) {
      __threadfence();
      ticket = atomicAdd(a.groups_done, 1u);
    }
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    if (ticket == gridDim.x - 1) {
      __threadfence();
      float part = 0.f;
      for (int i = lane; i < (int)gridDim.x; i += 32)
        part += *reinterpret_cast<volatile const float*>(a.loss_per_group + i);
      for (int s = 16; s > 0; s >>= 1) part += __shfl_xor_sync(0xffffffffu, part, s);
      if (lane == 0) *a.loss_mean = part * a.inv_groups_total;
    }
  }
}

typedef CUresult (*GateEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                 const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

GateEncodeFn gate_encode_fn() {
  static GateEncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<GateEncodeFn>(p);
  }
  return fn;
}

// [rows, m] bf16 row-major as a 3-D map {m, rows, 1} with a {64, box_rows, 1} box.
int gate_encode(CUtensorMap* map, const void* base, long long m, long long rows, int box_rows,
                const char* what) {
  GateEncodeFn fn = gate_encode_fn();
  if (!fn) return fail(MTFC_ERR_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
  cuuint64_t dims[3] = {(cuuint64_t)m, (cuuint64_t)rows, 1};
  cuuint64_t strides[2] = {(cuuint64_t)(m * 2), (cuuint64_t)(m * 2 * rows)};
  cuuint32_t box[3] = {(cuuint32_t)GBK, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MTFC_ERR_SHAPE, "tensor map for %s rejected (CUresult %d): m=%lld rows=%lld", what,
                (int)r, m, rows);
  return MTFC_OK;
}

// Launches `kernel` so that it may start while the previous kernel of the stream is
// still running (the kernel itself waits before it touches global memory).  If the
// attribute is refused the launch is repeated as an ordinary one.
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapping(void (*kernel)(KArgs...), unsigned grid, unsigned block, size_t smem,
                               cudaStream_t s, Args&&... args) {
  static bool refused = false;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = refused ? 0 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
  if (e != cudaSuccess && !refused) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(s, &cap);
    if (cap != cudaStreamCaptureStatusNone) return e;   // a failed capture cannot be retried here
    (void)cudaGetLastError();
    refused = true;
    cfg.numAttrs = 0;
    e = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
  }
  return e;
}

int padded_experts(int experts) { return experts <= 16 ? 16 : (experts <= 32 ? 32 : 64); }

int gate_stages(int ep, int r) {
  const int per_stage = r * X_STAGE_BYTES + 3 * ep * GBK * 2;
  int st = (200 * 1024) / per_stage;
  return st > MAX_STAGES ? MAX_STAGES : st;
}

size_t gate_fused_smem(int ep, int r) {
  return (size_t)gate_stages(ep, r) * (r * X_STAGE_BYTES + 3 * ep * GBK * 2) + 2 * G_EPI_WARPS * ep * 4 +
         2 * 2 * G_EPI_WARPS * ep * 4 + (2 * MAX_STAGES + 4) * 8 + 16 + 1024;
}

template <int EP, int R>
int launch_gate_fused(const CUtensorMap& mx, const CUtensorMap& mw, const GateFusedArgs& a,
                      cudaStream_t s) {
  static bool attr_set[64] = {false};
  int dev = 0;
  MTFC_CUDA(cudaGetDevice(&dev));
  const size_t smem = gate_fused_smem(EP, R);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    MTFC_CUDA(cudaFuncSetAttribute(gate_top2_fused<EP, R>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)smem));
    attr_set[dev] = true;
  }
  const int sms = sm_count();
  const unsigned grid = (unsigned)(a.num_tiles < sms ? a.num_tiles : sms);
  MTFC_CUDA(launch_overlapping(gate_top2_fused<EP, R>, grid, G_THREADS, smem, s, mx, mw, a));
  MTFC_LAUNCH_CHECK("gate_top2_fused");
  return MTFC_OK;
}

}  // namespace
}  // namespace mtfc

using namespace mtfc;

extern "C" {

int mtfc_moe_gate_fused_supported(int64_t m, int32_t experts) {
  return (m >= 8 && m % 8 == 0 && experts >= 2 && experts <= kMaxGateExperts) ? 1 : 0;
}

int32_t mtfc_moe_gate_padded_experts(int32_t experts) { return padded_experts(experts); }

int64_t mtfc_moe_gate_scratch_bytes(int64_t groups, int32_t group_size, int32_t experts) {
  if (groups < 0 || group_size < 1 || experts < 1) return 0;
  const int64_t tpg = (group_size + 63) / 64;   // the smaller of the two tile sizes
  // per tile: column sums of the raw gates (float) and two rows of counts (int)
  return groups * tpg * padded_experts(experts) * 4 * 3 + 16;
}

int mtfc_moe_gate_prepare(const float* w, int64_t m, int32_t experts, void* w3t_bf16, void* stream) {
  if (!w || !w3t_bf16 || m < 1 || experts < 1 || experts > kMaxGateExperts)
    return fail(MTFC_ERR_SHAPE, "gate_prepare: bad arguments");
  const int ep = padded_experts(experts);
  split_gate_weights_kmajor_kernel<<<grid_for(m * ep, 256), 256, 0,
                                     static_cast<cudaStream_t>(stream)>>>(
      w, m, experts, ep, static_cast<__nv_bfloat16*>(w3t_bf16));
  MTFC_LAUNCH_CHECK("split_gate_weights_kmajor_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_moe_gate_top2(const void* x_bf16, const void* w3t_bf16, int64_t groups, int32_t group_size,
                       int64_t m, int32_t experts, int32_t capacity, int32_t policy,
                       float threshold, const float* noise, int32_t* idx1, int32_t* idx2,
                       int32_t* pos1, int32_t* pos2, float* gate1, float* gate2, float* raw_gates,
                       float* loss_per_group, float* loss_mean, int64_t num_groups_total,
                       int32_t* slot_table, int32_t round_gates_to_bf16, void* scratch,
                       int64_t scratch_bytes, void* stream) {
  if (!x_bf16 || !w3t_bf16 || !idx1 || !idx2 || !pos1 || !pos2 || !gate1 || !gate2 ||
      !loss_per_group || !scratch)
    return fail(MTFC_ERR_SHAPE, "gate_top2: null argument");
  if (groups < 0 || group_size < 1 || capacity < 0)
    return fail(MTFC_ERR_SHAPE, "gate_top2: bad extents");
  if (!mtfc_moe_gate_fused_supported(m, experts))
    return fail(MTFC_ERR_UNSUPPORTED,
                "gate_top2: needs d_model a multiple of 8 and 2..%d experts (got %lld, %d)",
                kMaxGateExperts, (long long)m, experts);
  if (policy == MTFC_MOE_POLICY_RANDOM && !noise)
    return fail(MTFC_ERR_SHAPE, "gate_top2: policy random needs the noise tensor");
  if (policy < MTFC_MOE_POLICY_ALL || policy > MTFC_MOE_POLICY_SWITCH)
    return fail(MTFC_ERR_SHAPE, "gate_top2: unknown policy %d", policy);
  if ((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(w3t_bf16)) % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "gate_top2: buffers must be 16-byte aligned");
  if (groups == 0) return MTFC_OK;
  const long long tokens = groups * group_size;
  if (groups > INT32_MAX || tokens > INT32_MAX)
    return fail(MTFC_ERR_SHAPE, "gate_top2: too many tokens");
  if (scratch_bytes < mtfc_moe_gate_scratch_bytes(groups, group_size, experts))
    return fail(MTFC_ERR_SHAPE, "gate_top2: scratch of %lld bytes is too small", (long long)scratch_bytes);
  if ((long long)experts * capacity > INT32_MAX)
    return fail(MTFC_ERR_SHAPE, "gate_top2: experts*capacity too large");
  const int ep = padded_experts(experts);
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  GateFusedArgs a;
  a.group_size = group_size;
  a.experts = experts;
  a.m = (int)m;
  a.renormalize = policy != MTFC_MOE_POLICY_SWITCH;
  // 64-token tiles only when 128-token tiles would leave SMs without any tile: a
  // half-height tile halves the bytes a CTA keeps in flight, which costs more than
  // an uneven last round does
  const long long t128 = groups * ((group_size + 127) / 128);
  a.tile_rows = t128 < sm_count() ? 64 : 128;
  a.tiles_per_group = (group_size + a.tile_rows - 1) / a.tile_rows;
  // Tiles per pass over the gate kernel.  The kernel can take two (their accumulators
  // fit side by side for up to 32 experts), which halves the gate kernel's L2 reads;
  // on the 65536-token, 32-expert shape that measured slower (36.5 us against 32.1 us:
  // the pass's two epilogues run one after the other and the last one is exposed), so
  // every shape takes one.
  const int r = 1;
  a.big_per_group = (a.tiles_per_group + r - 1) / r;
  a.num_tiles = groups * a.big_per_group;
  a.stages = gate_stages(ep, r);

  CUtensorMap map_x, map_w;
  int rc = gate_encode(&map_x, x_bf16, m, tokens, a.tile_rows, "gate activations");
  if (rc != MTFC_OK) return rc;
  rc = gate_encode(&map_w, w3t_bf16, m, 3 * ep, 3 * ep, "gate kernel");
  if (rc != MTFC_OK) return rc;
  a.idx1 = idx1; a.idx2 = idx2; a.gate1 = gate1; a.gate2 = gate2;
  a.raw_gates = raw_gates;
  a.tile_sums = static_cast<float*>(scratch);
  a.tile_counts = reinterpret_cast<int*>(a.tile_sums + groups * a.tiles_per_group * ep);
  a.rank1 = pos1;
  a.rank2 = pos2;
  a.policy = policy;
  a.threshold = threshold;
  a.noise = noise;
  if ((long long)a.tiles_per_group * experts > 8192)
    return fail(MTFC_ERR_UNSUPPORTED, "gate_top2: group of %d tokens with %d experts is too long "
                "for the single-pass kernel; use the three-call form", group_size, experts);
  a.groups_done = reinterpret_cast<unsigned*>(
      static_cast<uint8_t*>(scratch) + mtfc_moe_gate_scratch_bytes(groups, group_size, experts) - 16);
  a.status = device_status_word();
  switch (ep) {
    case 16: rc = launch_gate_fused<16, 1>(map_x, map_w, a, s); break;
    case 32: rc = launch_gate_fused<32, 1>(map_x, map_w, a, s); break;
    default: rc = launch_gate_fused<64, 1>(map_x, map_w, a, s); break;
  }
  if (rc != MTFC_OK) return rc;

  PositionArgs p;
  p.group_size = group_size; p.experts = experts; p.capacity = capacity;
  p.idx1 = idx1; p.idx2 = idx2; p.pos1 = pos1; p.pos2 = pos2; p.gate1 = gate1; p.gate2 = gate2;
  p.tile_sums = a.tile_sums; p.tile_counts = a.tile_counts;
  p.tiles_per_group = a.tiles_per_group; p.tile_rows = a.tile_rows; p.ep = ep;
  p.loss_per_group = loss_per_group;
  p.loss_mean = loss_mean;
  p.inv_groups_total = 1.0f / (float)(num_groups_total > 0 ? num_groups_total : groups);
  p.groups_done = a.groups_done;
  p.table = slot_table;
  p.round_bf16 = round_gates_to_bf16;
  int threads = 1024;
  while (threads > 32 && threads / 2 >= group_size) threads >>= 1;
  const size_t base_smem = (size_t)(3 * a.tiles_per_group * experts + experts) * sizeof(int);
  const size_t table_smem = (size_t)experts * capacity * sizeof(int);
  p.table_in_smem = slot_table && base_smem + table_smem <= 96 * 1024;
  const size_t smem = base_smem + (p.table_in_smem ? table_smem : 0);
  if (smem > 48 * 1024) {
    static bool attr_set[64] = {false};
    int dev = 0;
    MTFC_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
      MTFC_CUDA(cudaFuncSetAttribute(top2_positions_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
      attr_set[dev] = true;
    }
  }
  MTFC_CUDA(launch_overlapping(top2_positions_kernel, (unsigned)groups, (unsigned)threads, smem, s, p));
  MTFC_LAUNCH_CHECK("top2_positions_kernel");
  count_launch(2);
  return MTFC_OK;
}

}  // extern "C"
