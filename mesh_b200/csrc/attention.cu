// K6 attn_fwd: softmax(q.k^T + causal bias).v for bf16 q/k/v without ever
// materialising the [batch, heads, length, memory_length] logits.
//
// Replaces the op chain of dot_product_attention
// (mesh_tensorflow/layers.py:1640-1652; transformer/attention.py:71-88):
// logits einsum, additive mask, fp32 softmax, cast of the weights to v.dtype,
// weighted-sum einsum.  The causal bias of the reference is an additive -1e9 on
// fp32 logits (layers.py:1839-1850): the logit is absorbed and exp() of it
// underflows to exactly 0, so masked keys contribute nothing and key blocks
// wholly to the right of a query block are skipped.
//
// One CTA handles 128 query rows of one (batch, head): 6 warps.
//   warp 0 lane 0 : TMA producer - Q once, then K and V blocks of 128 keys into
//                   two-stage rings (4-D tensor maps, so [b,h,l,d] and [b,l,h,d]
//                   are both read in place)
//   warp 1 lane 0 : MMA issuer   - S_j = Q.K_j^T (tcgen05, fp32 in TMEM, two S
//                   buffers) and O += P_j.V_j (O in TMEM); S_{j+1} is issued
//                   before softmax_j finishes, so the tensor core and the
//                   softmax overlap
//   warps 2..5    : softmax      - one query row per thread: running max and sum
//                   in fp32, P_j written to shared memory as the bf16 A operand
//                   of the second MMA, O rescaled in TMEM only when a row's max
//                   moved; at the end O / sum -> bf16 -> TMA store.
// All mbarrier waits are bounded (see tcgen05_ptx.cuh).

#include "tcgen05_ptx.cuh"

namespace mtfc {
namespace {

constexpr int ABM = 128;  // query rows per CTA
constexpr int ABN = 128;  // keys per block
constexpr int ATHREADS = 192;
constexpr int ATOM_BYTES = 128 * 128;  // 128 rows x 64 bf16 (one swizzle atom column)

struct AttnArgs {
  int lq, lk, heads, batch;
  int causal;
  float scale_log2e;  // softmax scale * log2(e)
  int* status;
};

constexpr float RESCALE_SLACK = 8.0f;

// Keeps sixteen registers' values where they are in program order: arithmetic on
// them cannot be moved above this point (no instruction is emitted).
__device__ __forceinline__ void pin16(uint32_t* r) {
  asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]),
                    "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]),
                    "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]));
}

// max(a, b, c) in one instruction.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Sets the logits of masked keys (past the end of the keys, or after the query
// under the causal mask) to -inf.  One compare and one select per logit, no
// branches: the last visible key is a per-thread number and the key offsets are
// compile-time constants.
__device__ __forceinline__ void mask_row(uint32_t (&sv)[4][32], int k0, int q_pos,
                                         const AttnArgs& args) {
  int last = args.lk - 1;
  if (args.causal) last = min(last, q_pos);
  const int last_rel = last - k0;
#pragma unroll
  for (int c = 0; c < 4; ++c)
#pragma unroll
    for (int i = 0; i < 32; ++i) sv[c][i] = (c * 32 + i > last_rel) ? 0xff800000u : sv[c][i];
}

// Maximum of a 128-logit row: four independent chains of 3-input maxima.
__device__ __forceinline__ float row_max(const uint32_t (&sv)[4][32]) {
  float mx[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    mx[c] = fmaxf(__uint_as_float(sv[c][0]), __uint_as_float(sv[c][1]));
#pragma unroll
    for (int i = 2; i < 32; i += 2)
      mx[c] = fmax3(mx[c], __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1]));
  }
  return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tc_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tc_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}
// Eight columns at a time, for the rarely taken output rescale, which runs while a
// whole row of logits is live in registers.
__device__ __forceinline__ void tc_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_st_32x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7])
      : "memory");
}

// kind::f16 instruction descriptor, fp32 accumulate, bf16 operands, M = 128.
__device__ __forceinline__ uint32_t attn_idesc(int n, int b_mn_major) {
  uint32_t d = 0;
  d |= 1u << 4;
  d |= 1u << 7;
  d |= 1u << 10;
  d |= (uint32_t)(b_mn_major & 1) << 16;
  d |= (uint32_t)(n >> 3) << 17;
  d |= (uint32_t)(ABM >> 4) << 24;
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Shared memory (D = head size, DA = D / 64 swizzle atoms of 64 columns):
//   Q  : DA atoms [128 rows][128 B]
//   K  : 2 stages x DA atoms         V : 2 stages x DA atoms
//   P  : 2 atoms (keys 0-63, 64-127) [128 rows][128 B]; reused to stage O
template <int D>
struct AttnSmem {
  static constexpr int DA = D / 64;
  static constexpr int Q = 0;
  static constexpr int K = Q + DA * ATOM_BYTES;
  static constexpr int V = K + 2 * DA * ATOM_BYTES;
  static constexpr int P = V + 2 * DA * ATOM_BYTES;
  static constexpr int BAR = P + 2 * ATOM_BYTES;
  static constexpr int NUM_BARS = 13;
  static constexpr int MISC = BAR + NUM_BARS * 8;
  static constexpr int USED = MISC + 16;
  static constexpr int ALLOC = USED + 1024;
};

template <int D>
__global__ void __launch_bounds__(ATHREADS, 1)
attn_fwd_tcgen05(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                 const AttnArgs args) {
  using SM = AttnSmem<D>;
  constexpr int DA = SM::DA;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + SM::BAR;
  // barrier indices
  const uint32_t q_full = bar_base;
  auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar_base + 8u * (3 + s); };
  auto v_full = [&](int s) { return bar_base + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar_base + 8u * (7 + s); };
  auto s_full = [&](int b) { return bar_base + 8u * (9 + b); };
  const uint32_t p_full = bar_base + 8u * 11;
  const uint32_t pv_done = bar_base + 8u * 12;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + SM::MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::MISC + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // heaviest (last) query blocks first under the causal mask
  const int num_qb = (args.lq + ABM - 1) / ABM;
  const int qb = num_qb - 1 - (int)blockIdx.x;
  const int head = blockIdx.y;
  const int bat = blockIdx.z;
  const int q0 = qb * ABM;
  int kv_len = args.lk;
  if (args.causal) kv_len = min(kv_len, q0 + ABM);
  const int num_kv = (kv_len + ABN - 1) / ABN;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
      mbar_init(s_full(s), 1);
    }
    mbar_init(p_full, 4);   // one arrival per softmax warp
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_base + SM::MISC),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s0 = tmem_base;             // S buffers: columns [0,128) and [128,256)
  const uint32_t tmem_o = tmem_base + 2 * ABN;    // O: columns [256, 256 + D)

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(q_full, DA * ATOM_BYTES);
#pragma unroll
      for (int a = 0; a < DA; ++a)
        tma_load_4d(smem_base + SM::Q + a * ATOM_BYTES, &map_q, q_full, a * 64, q0, head, bat);
      for (int j = 0; j < num_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        if (!mbar_wait(k_empty(st), ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_expect_tx(k_full(st), DA * ATOM_BYTES);
#pragma unroll
        for (int a = 0; a < DA; ++a)
          tma_load_4d(smem_base + SM::K + (st * DA + a) * ATOM_BYTES, &map_k, k_full(st), a * 64,
                      j * ABN, head, bat);
        if (!mbar_wait(v_empty(st), ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_expect_tx(v_full(st), DA * ATOM_BYTES);
#pragma unroll
        for (int a = 0; a < DA; ++a)
          tma_load_4d(smem_base + SM::V + (st * DA + a) * ATOM_BYTES, &map_v, v_full(st), a * 64,
                      j * ABN, head, bat);
      }
      if (!ok && args.status) atomicExch(args.status, MTFC_ERR_TIMEOUT);
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = attn_idesc(ABN, 0);  // Q (K-major) x K (K-major)
      const uint32_t idesc_o = attn_idesc(D, 1);    // P (K-major) x V (N-major)
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_s = [&](int j) {
        const int st = j & 1;
        const uint32_t d_tmem = tmem_s0 + (uint32_t)(st * ABN);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * ATOM_BYTES + (ks % 4) * 32;
          const uint64_t da = make_smem_desc(smem_base + SM::Q + off, 16, 1024);
          const uint64_t db = make_smem_desc(smem_base + SM::K + st * DA * ATOM_BYTES + off, 16, 1024);
          tc_mma_bf16(d_tmem, da, db, idesc_s, ks != 0 ? 1u : 0u);
        }
        tc_commit(k_empty(st));
        tc_commit(s_full(st));
      };
      if (ok && num_kv > 0) {
        ok = mbar_wait(k_full(0), 0, abort_flag);
        if (ok) { tc_fence_after(); issue_s(0); }
      }
      for (int j = 0; j < num_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        if (j + 1 < num_kv) {
          // S buffer (j+1)&1 was last read by softmax j-1, which finished before
          // it signalled p_full for block j-1 — already waited for below.
          if (!mbar_wait(k_full((j + 1) & 1), (uint32_t)(((j + 1) >> 1) & 1), abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_s(j + 1);
        }
        if (!mbar_wait(p_full, (uint32_t)(j & 1), abort_flag)) { ok = false; break; }
        if (!mbar_wait(v_full(st), ph, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < ABN / 16; ++ks) {
          const uint64_t da = make_smem_desc(
              smem_base + SM::P + (ks / 4) * ATOM_BYTES + (ks % 4) * 32, 16, 1024);
          const uint64_t db = make_smem_desc(
              smem_base + SM::V + st * DA * ATOM_BYTES + ks * 16 * 128, ATOM_BYTES, 1024);
          tc_mma_bf16(tmem_o, da, db, idesc_o, (j | ks) != 0 ? 1u : 0u);
        }
        tc_commit(v_empty(st));
        tc_commit(pv_done);
      }
      if (!ok && args.status) atomicExch(args.status, MTFC_ERR_TIMEOUT);
    }
  } else {
    // ------------------------------------------------- softmax / correction / output
    const int q = warp & 3;
    const int row = q * 32 + lane;          // query row of this thread inside the block
    const int q_pos = q0 + row;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < num_kv && ok; ++j) {
      const int st = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(s_full(st), (uint32_t)((j >> 1) & 1), abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_s = tmem_s0 + lane_base + (uint32_t)(st * ABN);
      const int k0 = j * ABN;
      const bool need_mask = (args.causal && k0 + ABN - 1 > q0) || (k0 + ABN > args.lk);
      // the whole S row into registers (four loads in flight, one wait), masked in
      // place, and its maximum (four independent chains; the scale is positive,
      // so it is applied to the maximum instead of to every logit)
      uint32_t sv[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tc_ld_32x32(t_s + c * 32, sv[c]);
      tc_wait_ld();
      if (need_mask) mask_row(sv, k0, q_pos, args);
      const float m_blk = row_max(sv) * args.scale_log2e;
      const float m_new = fmaxf(m_run, m_blk);
      // a fully masked row (only possible for rows past the end) keeps m = -inf
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_use);
      // P_{j-1} and O are free once the previous P.V has retired
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(pv_done, (uint32_t)((j - 1) & 1), abort_flag));
        if (!ok) break;
        tc_fence_after();
        const bool rescale = __any_sync(0xffffffffu, alpha != 1.0f);
        if (rescale) {
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t v[32];
            tc_ld_32x32(tmem_o + lane_base + c, v);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tc_st_32x32(tmem_o + lane_base + c, v);
          }
          tc_wait_st();
        }
      }
      // p = 2^(scale * s - m), row sum, bf16 P into the swizzled A-operand tile
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
      uint8_t* p_row = smem + SM::P + row * 128;
      const int sw = row & 7;
      const float neg_m = -m_use;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float p[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          // masked logits are -inf: 2^(-inf) = 0
          p[i] = fast_exp2(fmaf(__uint_as_float(sv[c][i]), args.scale_log2e, neg_m));
          ls[i & 3] += p[i];
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o;
          o.x = pack_bf16x2(p[8 * g + 0], p[8 * g + 1]);
          o.y = pack_bf16x2(p[8 * g + 2], p[8 * g + 3]);
          o.z = pack_bf16x2(p[8 * g + 4], p[8 * g + 5]);
          o.w = pack_bf16x2(p[8 * g + 6], p[8 * g + 7]);
          const int chunk = c * 4 + g;             // 16-byte chunk index along the 128 keys
          const int atom = chunk >> 3, cc = chunk & 7;
          *reinterpret_cast<uint4*>(p_row + atom * ATOM_BYTES + ((cc ^ sw) << 4)) = o;
        }
      }
      const float l_blk = (ls[0] + ls[1]) + (ls[2] + ls[3]);
      l_run = l_run * alpha + l_blk;
      m_run = m_new;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- output: O / l -> bf16 -> staging (P tile) -> TMA store
    if (ok && num_kv > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(pv_done, (uint32_t)((num_kv - 1) & 1), abort_flag));
    }
    if (ok) {
      tc_fence_after();
      const float inv_l = l_run > 0.f ? 1.0f / l_run : 0.f;
      uint8_t* o_row = smem + SM::P + q * 32 * 128 + lane * 128;  // this warp's 32 rows per atom
      const int sw = lane & 7;
      if ((q0 + q * 32) < args.lq) {
#pragma unroll 1
        for (int a = 0; a < DA; ++a) {
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            uint32_t v[32];
            if (num_kv > 0) {
              tc_ld_32x32(tmem_o + lane_base + a * 64 + h * 32, v);
              tc_wait_ld();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = 0u;
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[8 * g + 0]) * inv_l, __uint_as_float(v[8 * g + 1]) * inv_l);
              o.y = pack_bf16x2(__uint_as_float(v[8 * g + 2]) * inv_l, __uint_as_float(v[8 * g + 3]) * inv_l);
              o.z = pack_bf16x2(__uint_as_float(v[8 * g + 4]) * inv_l, __uint_as_float(v[8 * g + 5]) * inv_l);
              o.w = pack_bf16x2(__uint_as_float(v[8 * g + 6]) * inv_l, __uint_as_float(v[8 * g + 7]) * inv_l);
              *reinterpret_cast<uint4*>(o_row + a * ATOM_BYTES + (((h * 4 + g) ^ sw) << 4)) = o;
            }
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
#pragma unroll 1
          for (int a = 0; a < DA; ++a)
            tma_store_4d(&map_o, smem_base + SM::P + a * ATOM_BYTES + q * 32 * 128, a * 64,
                         q0 + q * 32, head, bat);
          tma_store_commit();
          tma_store_wait_all();
        }
      }
    }
    if (!ok && lane == 0 && args.status) atomicExch(args.status, MTFC_ERR_TIMEOUT);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512)
                 : "memory");
  }
}

// ------------------------------------------------------------ two-tile variant
// Two query tiles (A, B: 2 x 128 rows of one (batch, head)) per CTA, each with
// its own warpgroup of four softmax warps, sharing every K / V block.  The MMA
// issuer alternates S_A, S_B, P_A.V, P_B.V so that one tile's softmax always
// overlaps the other tile's tensor-core work, and there are two softmax warps
// per scheduler instead of one.  P never touches shared memory: the bf16 weights
// are stored back into TMEM over the first 64 columns of their S tile and feed
// the second MMA as its A operand from TMEM.
// TMEM columns: S_A/P_A [0,128)  S_B/P_B [128,256)  O_A [256,256+D)  O_B [384,384+D).
constexpr int A2THREADS = 352;

template <int D>
struct Attn2Smem {
  static constexpr int DA = D / 64;
  static constexpr int Q = 0;                              // 2 tiles x DA atoms
  static constexpr int K = Q + 2 * DA * ATOM_BYTES;        // 2 stages x DA atoms
  static constexpr int V = K + 2 * DA * ATOM_BYTES;        // 2 stages x DA atoms
  static constexpr int BAR = V + 2 * DA * ATOM_BYTES;
  static constexpr int NUM_BARS = 20;
  static constexpr int MISC = BAR + NUM_BARS * 8;
  static constexpr int USED = MISC + 16;
  static constexpr int ALLOC = USED + 1024;
};

__device__ __forceinline__ void tc_mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int D>
__global__ void __launch_bounds__(A2THREADS, 1)
attn_fwd_tcgen05_2tile(const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v,
                       const __grid_constant__ CUtensorMap map_o, const AttnArgs args) {
  using SM = Attn2Smem<D>;
  constexpr int DA = SM::DA;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + SM::BAR;
  const uint32_t q_full = bar_base;
  auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar_base + 8u * (3 + s); };
  auto v_full = [&](int s) { return bar_base + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar_base + 8u * (7 + s); };
  auto s_full = [&](int t) { return bar_base + 8u * (9 + t); };    // per tile
  auto pv_done = [&](int t) { return bar_base + 8u * (11 + t); };  // per tile
  // weights of keys 0-63 (h = 0) and 64-127 (h = 1) of a tile stored to TMEM
  auto p_half = [&](int t, int h) { return bar_base + 8u * (13 + 2 * t + h); };
  auto exp_done = [&](int t) { return bar_base + 8u * (17 + t); };  // tile t finished a block's exponentials
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + SM::MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SM::MISC + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_qb = (args.lq + 2 * ABM - 1) / (2 * ABM);
  const int qb = num_qb - 1 - (int)blockIdx.x;  // heaviest blocks first under the causal mask
  const int head = blockIdx.y;
  const int bat = blockIdx.z;
  const int q0 = qb * 2 * ABM;
  // key blocks each tile needs (tile B sits 128 rows lower, so one more when causal)
  int n_tile[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    int kv_len = args.lk;
    if (args.causal) kv_len = min(kv_len, q0 + t * ABM + ABM);
    n_tile[t] = (q0 + t * ABM < args.lq) ? (kv_len + ABN - 1) / ABN : 0;
  }
  const int num_kv = max(n_tile[0], n_tile[1]);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 2);   // one arrival per MMA issuer
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 2);
      mbar_init(s_full(s), 1);
      mbar_init(p_half(s, 0), 4);
      mbar_init(p_half(s, 1), 4);
      mbar_init(pv_done(s), 1);
      mbar_init(exp_done(s), 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_base + SM::MISC),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  auto tmem_s = [&](int t) { return tmem_base + (uint32_t)(t * ABN); };
  auto tmem_o = [&](int t) { return tmem_base + (uint32_t)(2 * ABN + t * 128); };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      mbar_expect_tx(q_full, 2 * DA * ATOM_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int a = 0; a < DA; ++a)
          tma_load_4d(smem_base + SM::Q + (t * DA + a) * ATOM_BYTES, &map_q, q_full, a * 64,
                      q0 + t * ABM, head, bat);
      for (int j = 0; j < num_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        if (!mbar_wait(k_empty(st), ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_expect_tx(k_full(st), DA * ATOM_BYTES);
#pragma unroll
        for (int a = 0; a < DA; ++a)
          tma_load_4d(smem_base + SM::K + (st * DA + a) * ATOM_BYTES, &map_k, k_full(st), a * 64,
                      j * ABN, head, bat);
        if (!mbar_wait(v_empty(st), ph ^ 1, abort_flag)) { ok = false; break; }
        mbar_expect_tx(v_full(st), DA * ATOM_BYTES);
#pragma unroll
        for (int a = 0; a < DA; ++a)
          tma_load_4d(smem_base + SM::V + (st * DA + a) * ATOM_BYTES, &map_v, v_full(st), a * 64,
                      j * ABN, head, bat);
      }
      if (!ok && args.status) atomicExch(args.status, MTFC_ERR_TIMEOUT);
    }
  } else if (warp == 1 || warp == 10) {
    // ------------------------------------------- MMA issuers, one thread per tile
    // Each tile's products are issued in order by its own thread, so the tensor
    // pipe interleaves the two tiles by itself and neither tile's issue ever waits
    // on the other tile's softmax.  K / V stages are released by both threads.
    if (lane == 0) {
      const int t = warp == 1 ? 0 : 1;
      const int n_mine = n_tile[t];
      const uint32_t idesc_s = attn_idesc(ABN, 0);
      const uint32_t idesc_o = attn_idesc(D, 1);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_s = [&](int j) {   // S_t(j) = Q_t . K_j^T
        const int st = j & 1;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks / 4) * ATOM_BYTES + (ks % 4) * 32;
          const uint64_t da = make_smem_desc(smem_base + SM::Q + t * DA * ATOM_BYTES + off, 16, 1024);
          const uint64_t db = make_smem_desc(smem_base + SM::K + st * DA * ATOM_BYTES + off, 16, 1024);
          tc_mma_bf16(tmem_s(t), da, db, idesc_s, ks != 0 ? 1u : 0u);
        }
        tc_commit(s_full(t));
      };
      auto issue_pv_half = [&](int j, int h) {  // O_t += P_t(j)[:, 64h:64h+64] . V_j[64h:64h+64], P from TMEM
        const int st = j & 1;
#pragma unroll
        for (int kk = 0; kk < ABN / 32; ++kk) {
          const int ks = h * (ABN / 32) + kk;
          const uint64_t db = make_smem_desc(
              smem_base + SM::V + st * DA * ATOM_BYTES + ks * 16 * 128, ATOM_BYTES, 1024);
          tc_mma_bf16_ts(tmem_o(t), tmem_s(t) + (uint32_t)(ks * 8), db, idesc_o,
                         (j | ks) != 0 ? 1u : 0u);
        }
      };
      if (ok && num_kv > 0) {
        ok = mbar_wait(k_full(0), 0, abort_flag);
        if (ok) {
          tc_fence_after();
          if (n_mine > 0) issue_s(0);
          tc_commit(k_empty(0));
        }
      }
      for (int j = 0; j < num_kv && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)((j >> 1) & 1);
        const bool next = j + 1 < num_kv;
        // waited for even when this tile skips the block, so that the two issuers
        // release a stage exactly once each per block
        if (!mbar_wait(v_full(st), ph, abort_flag)) { ok = false; break; }
        if (next && !mbar_wait(k_full((j + 1) & 1), (uint32_t)(((j + 1) >> 1) & 1), abort_flag)) {
          ok = false;
          break;
        }
        if (j < n_mine) {
          if (!mbar_wait(p_half(t, 0), (uint32_t)(j & 1), abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_pv_half(j, 0);
          if (!mbar_wait(p_half(t, 1), (uint32_t)(j & 1), abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_pv_half(j, 1);
          tc_commit(pv_done(t));
          // the tensor pipe runs this thread's MMAs in order, so S_t(j+1) may
          // overwrite the columns P_t(j) occupies as soon as P.V is queued
          if (j + 1 < n_mine) issue_s(j + 1);
        }
        tc_commit(v_empty(st));
        if (next) tc_commit(k_empty((j + 1) & 1));
      }
      if (!ok && args.status) atomicExch(args.status, MTFC_ERR_TIMEOUT);
    }
  } else {
    // ------------------------------------------------- softmax warpgroups (tile 0: warps 2-5, tile 1: 6-9)
    const int t = (warp - 2) >> 2;
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int q_pos = q0 + t * ABM + row;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const uint32_t t_s = tmem_s(t) + lane_base;
    const uint32_t t_o = tmem_o(t) + lane_base;
    const int n_mine = n_tile[t];
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_mine && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(s_full(t), (uint32_t)(j & 1), abort_flag));
      if (!ok) break;
      tc_fence_after();
      const int k0 = j * ABN;
      const bool need_mask = (args.causal && k0 + ABN - 1 > q0 + t * ABM) || (k0 + ABN > args.lk);
      uint32_t sv[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tc_ld_32x32(t_s + c * 32, sv[c]);
      tc_wait_ld();
      if (need_mask) mask_row(sv, k0, q_pos, args);
      const float m_blk = row_max(sv) * args.scale_log2e;
      // The running reference m_run only moves when the block maximum exceeds it
      // by more than RESCALE_SLACK (in log2 units): weights then reach at most
      // 2^RESCALE_SLACK, harmless in bf16 / fp32, the common factor cancels in O / l,
      // and O is rescaled in a small fraction of the blocks instead of nearly all.
      const bool moved = m_blk > m_run + RESCALE_SLACK;   // also true for m_run = -inf
      const float m_new = moved ? m_blk : m_run;
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = !moved ? 1.0f : ((m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_use));
      const float neg_m = -m_use;
      // O_t is rescaled (rarely) before any of this block's P.V is queued.  S_t(j)
      // was queued behind P.V(j-1), so that product has retired by now; the wait
      // only orders this thread's O accesses after it.
      if (j > 0 && __any_sync(0xffffffffu, moved)) {
        ok = __all_sync(0xffffffffu, mbar_wait(pv_done(t), (uint32_t)((j - 1) & 1), abort_flag));
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < D; c += 8) {
          uint32_t v[8];
          tc_ld_32x8(t_o + c, v);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tc_st_32x8(t_o + c, v);
        }
      }
      // bf16 weights, packed two per register, stored over the first 64 columns of
      // this tile's S region 64 keys at a time (S itself is already in registers,
      // and the previous P.V — which read these columns — retired before S_t(j) was
      // written), and the row sum.  Each half is handed to the MMA issuer as soon
      // as it is stored, so P.V starts on keys 0-63 while keys 64-127 are still
      // being exponentiated.
      //
      // The two tiles take turns at the exponentials (tile 0 block j, tile 1 block j,
      // tile 0 block j+1, ...): the special-function unit is the scarcest resource
      // of this loop (4 lanes per clock per scheduler, and a warp that runs into a
      // busy unit issues nothing else meanwhile), and two tiles exponentiating at
      // once would each run at half speed while the tensor pipe idles; in turns,
      // one tile's exponentials hide behind the other tile's products.  What needs
      // no special-function unit stays out of the turn: the scaling of the logits
      // is done before it (in the issue slots the other tile leaves free) and the
      // row sum after the weights have been handed over.
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i)
          sv[c][i] = __float_as_uint(fmaf(__uint_as_float(sv[c][i]), args.scale_log2e, neg_m));
      {
        const int n_other = n_tile[1 - t];
        bool turn = true;
        if (t == 0) {
          if (j > 0 && j - 1 < n_other) turn = mbar_wait(exp_done(1), (uint32_t)((j - 1) & 1), abort_flag);
        } else {
          if (j < n_other) turn = mbar_wait(exp_done(0), (uint32_t)(j & 1), abort_flag);
        }
        ok = __all_sync(0xffffffffu, turn);
        if (!ok) break;
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = fast_exp2(__uint_as_float(sv[2 * h + cc][i]));       // masked: 2^-inf = 0
            const float p1 = fast_exp2(__uint_as_float(sv[2 * h + cc][i + 1]));
            sv[2 * h + cc][i] = __float_as_uint(p0);
            sv[2 * h + cc][i + 1] = __float_as_uint(p1);
            pk[i >> 1] = pack_bf16x2(p0, p1);
          }
          tc_st_32x16(t_s + h * 32 + cc * 16, pk);
        }
        if (h == 1) {
          __syncwarp();
          if (lane == 0) mbar_arrive(exp_done(t));
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_half(t, h));
      }
      // row sum of the (unrounded) weights, while the tensor pipe works on them
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        pin16(&sv[c][0]);
        pin16(&sv[c][16]);
#pragma unroll
        for (int i = 0; i < 32; ++i) ls[i & 3] += __uint_as_float(sv[c][i]);
      }
      l_run = l_run * alpha + ((ls[0] + ls[1]) + (ls[2] + ls[3]));
      m_run = m_new;
    }
    if (ok && n_mine > 0)
      ok = __all_sync(0xffffffffu, mbar_wait(pv_done(t), (uint32_t)((n_mine - 1) & 1), abort_flag));
    if (ok && n_mine > 0) {
      // O / l -> bf16 -> this tile's Q region (no longer read: every S MMA of the
      // tile retired before its last P.V) -> TMA store
      tc_fence_after();
      const float inv_l = l_run > 0.f ? 1.0f / l_run : 0.f;
      uint8_t* o_row = smem + SM::Q + t * DA * ATOM_BYTES + q * 32 * 128 + lane * 128;
      const int sw = lane & 7;
      if ((q0 + t * ABM + q * 32) < args.lq) {
#pragma unroll 1
        for (int a = 0; a < DA; ++a) {
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            uint32_t v[32];
            tc_ld_32x32(t_o + a * 64 + h * 32, v);
            tc_wait_ld();
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(v[8 * g + 0]) * inv_l, __uint_as_float(v[8 * g + 1]) * inv_l);
              o.y = pack_bf16x2(__uint_as_float(v[8 * g + 2]) * inv_l, __uint_as_float(v[8 * g + 3]) * inv_l);
              o.z = pack_bf16x2(__uint_as_float(v[8 * g + 4]) * inv_l, __uint_as_float(v[8 * g + 5]) * inv_l);
              o.w = pack_bf16x2(__uint_as_float(v[8 * g + 6]) * inv_l, __uint_as_float(v[8 * g + 7]) * inv_l);
              *reinterpret_cast<uint4*>(o_row + a * ATOM_BYTES + (((h * 4 + g) ^ sw) << 4)) = o;
            }
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
#pragma unroll 1
          for (int a = 0; a < DA; ++a)
            tma_store_4d(&map_o, smem_base + SM::Q + (t * DA + a) * ATOM_BYTES + q * 32 * 128,
                         a * 64, q0 + t * ABM + q * 32, head, bat);
          tma_store_commit();
          tma_store_wait_all();
        }
      }
    }
    if (!ok && lane == 0 && args.status) atomicExch(args.status, MTFC_ERR_TIMEOUT);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512)
                 : "memory");
  }
}

}  // namespace
}  // namespace mtfc

namespace mtfc {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn attn_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 4-D bf16 map {d, length, heads, batch} with a {64, box_rows, 1, 1} box, 128B swizzle.
int attn_map(CUtensorMap* map, const void* base, int64_t d, int64_t len, int64_t heads,
             int64_t batch, int64_t s_len, int64_t s_head, int64_t s_batch, int box_rows,
             const char* what) {
  EncodeTiledFn fn = attn_encode_fn();
  if (!fn) return fail(MTFC_ERR_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
  cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)len, (cuuint64_t)heads, (cuuint64_t)batch};
  int64_t sl = s_len * 2, sh = s_head * 2, sb = s_batch * 2;
  if (len == 1 || sl <= 0) sl = ((d * 2 + 15) / 16) * 16;
  if (heads == 1 || sh <= 0) sh = sl * len;
  if (batch == 1 || sb <= 0) sb = sh * heads;
  cuuint64_t strides[3] = {(cuuint64_t)sl, (cuuint64_t)sh, (cuuint64_t)sb};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MTFC_ERR_SHAPE, "attention: tensor map for %s rejected (CUresult %d)", what, (int)r);
  return MTFC_OK;
}

template <int D>
int attn_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                const CUtensorMap& mo, const AttnArgs& args, cudaStream_t stream) {
  static bool attr_set[64] = {false};
  int dev = 0;
  MTFC_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    MTFC_CUDA(cudaFuncSetAttribute(attn_fwd_tcgen05<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   AttnSmem<D>::ALLOC));
    attr_set[dev] = true;
  }
  dim3 grid((unsigned)((args.lq + ABM - 1) / ABM), (unsigned)args.heads, (unsigned)args.batch);
  attn_fwd_tcgen05<D><<<grid, ATHREADS, AttnSmem<D>::ALLOC, stream>>>(mq, mk, mv, mo, args);
  MTFC_LAUNCH_CHECK("attn_fwd_tcgen05");
  return MTFC_OK;
}

template <int D>
int attn2_launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                 const CUtensorMap& mo, const AttnArgs& args, cudaStream_t stream) {
  static bool attr_set[64] = {false};
  int dev = 0;
  MTFC_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    MTFC_CUDA(cudaFuncSetAttribute(attn_fwd_tcgen05_2tile<D>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, Attn2Smem<D>::ALLOC));
    attr_set[dev] = true;
  }
  dim3 grid((unsigned)((args.lq + 2 * ABM - 1) / (2 * ABM)), (unsigned)args.heads,
            (unsigned)args.batch);
  attn_fwd_tcgen05_2tile<D><<<grid, A2THREADS, Attn2Smem<D>::ALLOC, stream>>>(mq, mk, mv, mo, args);
  MTFC_LAUNCH_CHECK("attn_fwd_tcgen05_2tile");
  return MTFC_OK;
}

int g_attn_variant = 0;  // 0 = choose by length, 1 = one tile per CTA, 2 = two tiles per CTA

}  // namespace
}  // namespace mtfc

using namespace mtfc;

extern "C" {

int mtfc_attention_set_variant(int variant) {
  if (variant < 0 || variant > 2) return fail(MTFC_ERR_SHAPE, "attention variant %d unknown", variant);
  g_attn_variant = variant;
  return MTFC_OK;
}

int mtfc_attention_supported(int64_t d, const int64_t* q_strides, const int64_t* k_strides,
                             const int64_t* v_strides, const int64_t* o_strides) {
  if (d != 64 && d != 128) return 0;
  const int64_t* all[4] = {q_strides, k_strides, v_strides, o_strides};
  for (int t = 0; t < 4; ++t) {
    if (!all[t]) return 0;
    if (all[t][3] != 1) return 0;                       // head dim contiguous
    for (int i = 0; i < 3; ++i)
      if (all[t][i] % 8 != 0) return 0;                 // 16-byte multiples for TMA
  }
  return 1;
}

int mtfc_attention_fwd(const void* q, const void* k, const void* v, void* out, int64_t batch,
                       int64_t heads, int64_t lq, int64_t lk, int64_t d, const int64_t* q_strides,
                       const int64_t* k_strides, const int64_t* v_strides,
                       const int64_t* o_strides, int32_t causal, float scale, void* stream) {
  if (!q || !k || !v || !out) return fail(MTFC_ERR_SHAPE, "attention: null argument");
  if (batch < 0 || heads < 0 || lq < 0 || lk < 1)
    return fail(MTFC_ERR_SHAPE, "attention: bad extents");
  if (!mtfc_attention_supported(d, q_strides, k_strides, v_strides, o_strides))
    return fail(MTFC_ERR_SHAPE,
                "attention: needs head size 64 or 128, a contiguous head dim and strides that are "
                "multiples of 8 elements");
  if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
        reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out)) & 15) != 0)
    return fail(MTFC_ERR_SHAPE, "attention: buffers must be 16-byte aligned");
  if (batch == 0 || heads == 0 || lq == 0) return MTFC_OK;
  if (heads > 65535 || batch > 65535) return fail(MTFC_ERR_SHAPE, "attention: grid too large");
  CUtensorMap mq, mk, mv, mo;
  int rc = attn_map(&mq, q, d, lq, heads, batch, q_strides[2], q_strides[1], q_strides[0], ABM, "q");
  if (rc != MTFC_OK) return rc;
  rc = attn_map(&mk, k, d, lk, heads, batch, k_strides[2], k_strides[1], k_strides[0], ABN, "k");
  if (rc != MTFC_OK) return rc;
  rc = attn_map(&mv, v, d, lk, heads, batch, v_strides[2], v_strides[1], v_strides[0], ABN, "v");
  if (rc != MTFC_OK) return rc;
  rc = attn_map(&mo, out, d, lq, heads, batch, o_strides[2], o_strides[1], o_strides[0], 32, "out");
  if (rc != MTFC_OK) return rc;
  AttnArgs args;
  args.lq = (int)lq;
  args.lk = (int)lk;
  args.heads = (int)heads;
  args.batch = (int)batch;
  args.causal = causal ? 1 : 0;
  args.scale_log2e = scale * 1.4426950408889634f;
  args.status = device_status_word();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool two_tiles = g_attn_variant == 2 || (g_attn_variant == 0 && lq > ABM);
  if (two_tiles)
    rc = d == 128 ? attn2_launch<128>(mq, mk, mv, mo, args, s) : attn2_launch<64>(mq, mk, mv, mo, args, s);
  else
    rc = d == 128 ? attn_launch<128>(mq, mk, mv, mo, args, s) : attn_launch<64>(mq, mk, mv, mo, args, s);
  if (rc == MTFC_OK) count_launch(1);
  return rc;
}

}  // extern "C"
