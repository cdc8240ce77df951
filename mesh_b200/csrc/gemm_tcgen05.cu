// K1 einsum_gemm: C[b,m,n] = epilogue(sum_k A[b,m,k] * B[b,k,n]) on the sm_100a
// tensor cores.  bf16 operands, fp32 accumulation in TMEM, bf16 or fp32 output.
//
// Replaces the per-slice tf.einsum of MeshImpl.einsum (mesh_tensorflow/ops.py:
// 1331-1340).  Either operand may be K-major (contracted dim contiguous) or
// MN-major (free dim contiguous): the shared-memory matrix descriptors and the
// instruction descriptor's major bits take the layout as it is, so the named
// dim order of a laid-out tensor never has to be transposed in memory.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0 lane 0 : TMA producer  - cp.async.bulk.tensor loads into a 4-stage
//                   ring of 128B-swizzled tiles (A 128x64, B 256x64 bf16)
//   warp 1 lane 0 : MMA issuer    - tcgen05.mma 128x256x16, accumulators in
//                   TMEM, two accumulator buffers (2 x 256 columns)
//   warps 2..5    : epilogue      - tcgen05.ld, ReLU/convert, swizzled staging
//                   in shared memory, TMA store (clipped at the M/N edges)
// so the epilogue of tile i overlaps the main loop of tile i+1.  No load uses
// cluster multicast.  Every mbarrier wait is bounded: on expiry the kernel
// raises a CTA-wide abort flag, records MTFC_ERR_TIMEOUT in the device status
// word, drains, frees its TMEM and returns.

#include <cstring>
#include "tcgen05_ptx.cuh"

namespace mtfc {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int MN_GROUP_BYTES = 64 * BK * 2;  // one 64(MN) x 64(K) box, 8 KiB
constexpr int EPI_WARPS = 4;
constexpr int EPI_BUF_BYTES = 32 * 128;  // 32 rows x 128 B per staging buffer
constexpr int EPI_BYTES = EPI_WARPS * 2 * EPI_BUF_BYTES;
constexpr int NUM_THREADS = 32 * (2 + EPI_WARPS);
constexpr int TMEM_COLS = 512;

constexpr int SMEM_A = 0;
constexpr int SMEM_B = SMEM_A + STAGES * A_STAGE_BYTES;
constexpr int SMEM_EPI = SMEM_B + STAGES * B_STAGE_BYTES;
constexpr int SMEM_BAR = SMEM_EPI + EPI_BYTES;
// barriers: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
constexpr int NUM_BARS = 2 * STAGES + 4;
constexpr int SMEM_MISC = SMEM_BAR + NUM_BARS * 8;  // tmem base (4 B) + abort flag (4 B)
constexpr int SMEM_USED = SMEM_MISC + 16;
constexpr int SMEM_ALLOC = SMEM_USED + 1024;  // slack for manual 1 KiB alignment


struct GemmArgs {
  int m, n, k, batch;
  int tiles_m, tiles_n;
  int a_mn_major, b_mn_major;
  int a_batched, b_batched;
  int relu;
  int out_f32;
  int* status;
  // pair kernel only, optional: progress[rb] is incremented once per epilogue warp
  // and tile of 256-row block rb when that tile's rows have landed in memory
  // (tiles_n * 8 increments complete a row block), for a consumer on another
  // stream that starts on row blocks while later ones are still being multiplied
  uint32_t* progress;
};

// Instruction descriptor for kind::f16: fp32 accumulator, bf16 A and B,
// major bits, N >> 3 at [17,23), M >> 4 at [24,29).
__device__ __forceinline__ uint32_t make_idesc(int a_mn, int b_mn) {
  uint32_t d = 0;
  d |= 1u << 4;   // D format fp32
  d |= 1u << 7;   // A format bf16
  d |= 1u << 10;  // B format bf16
  d |= (uint32_t)(a_mn & 1) << 15;
  d |= (uint32_t)(b_mn & 1) << 16;
  d |= (uint32_t)(BN >> 3) << 17;
  d |= (uint32_t)(BM >> 4) << 24;
  return d;
}


// ------------------------------------------------------------------ the kernel
__global__ void __launch_bounds__(NUM_THREADS, 1)
einsum_gemm_tcgen05(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_c, const GemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  // Swizzled tiles need 1 KiB alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + SMEM_BAR;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + SMEM_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + SMEM_MISC + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tmem_full_bar(b), 1);
      mbar_init(tmem_empty_bar(b), EPI_WARPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_base + SMEM_MISC),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_kb = (args.k + BK - 1) / BK;
  const long long tiles_per_batch = (long long)args.tiles_m * args.tiles_n;
  const long long num_tiles = tiles_per_batch * args.batch;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int b = (int)(t / tiles_per_batch);
        const int r = (int)(t % tiles_per_batch);
        const int m0 = (r / args.tiles_n) * BM;
        const int n0 = (r % args.tiles_n) * BN;
        const int ab = args.a_batched ? b : 0;
        const int bb = args.b_batched ? b : 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), A_STAGE_BYTES + B_STAGE_BYTES);
          const uint32_t sa = smem_base + SMEM_A + stage * A_STAGE_BYTES;
          const uint32_t sb = smem_base + SMEM_B + stage * B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (args.a_mn_major) {
#pragma unroll
            for (int g = 0; g < BM / 64; ++g)
              tma_load_3d(sa + g * MN_GROUP_BYTES, &map_a, full_bar(stage), m0 + g * 64, k0, ab);
          } else {
            tma_load_3d(sa, &map_a, full_bar(stage), k0, m0, ab);
          }
          if (args.b_mn_major) {
#pragma unroll
            for (int g = 0; g < BN / 64; ++g)
              tma_load_3d(sb + g * MN_GROUP_BYTES, &map_b, full_bar(stage), n0 + g * 64, k0, bb);
          } else {
            tma_load_3d(sb, &map_b, full_bar(stage), k0, n0, bb);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok && args.status) atomicExch(args.status, MTFC_ERR_TIMEOUT);
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc(args.a_mn_major, args.b_mn_major);
      const uint32_t a_lbo = args.a_mn_major ? MN_GROUP_BYTES : 16;
      const uint32_t b_lbo = args.b_mn_major ? MN_GROUP_BYTES : 16;
      // bytes to advance the start address per UMMA_K step inside a stage
      const uint32_t a_kstep = args.a_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_kstep = args.b_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long local = 0;
      for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
        const int buf = (int)(local & 1);
        const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
        if (!mbar_wait(tmem_empty_bar(buf), acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + SMEM_A + stage * A_STAGE_BYTES;
          const uint32_t sb = smem_base + SMEM_B + stage * B_STAGE_BYTES;
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks) {
            const uint64_t da = make_smem_desc(sa + ks * a_kstep, a_lbo, 1024);
            const uint64_t db = make_smem_desc(sb + ks * b_kstep, b_lbo, 1024);
            tc_mma_bf16(d_tmem, da, db, idesc, (kb | ks) != 0 ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));  // frees the stage once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(tmem_full_bar(buf));  // accumulator ready for the epilogue
      }
      if (!ok && args.status) atomicExch(args.status, MTFC_ERR_TIMEOUT);
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int ew = warp - 2;
    uint8_t* stage_buf = smem + SMEM_EPI + ew * 2 * EPI_BUF_BYTES;
    const uint32_t stage_u32 = smem_base + SMEM_EPI + ew * 2 * EPI_BUF_BYTES;
    const int cols_per_store = args.out_f32 ? 32 : 64;  // 128 B of output per row
    bool ok = true;
    long long local = 0;
    int store_idx = 0;
    for (long long t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
      const int buf = (int)(local & 1);
      const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
      const int b = (int)(t / tiles_per_batch);
      const int r = (int)(t % tiles_per_batch);
      const int m0 = (r / args.tiles_n) * BM;
      const int n0 = (r % args.tiles_n) * BN;
      // Warp-uniform outcome: the .sync.aligned TMEM loads below need all lanes.
      ok = __all_sync(0xffffffffu, mbar_wait(tmem_full_bar(buf), acc_phase, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
      const bool rows_live = (m0 + q * 32) < args.m;
      for (int c0 = 0; c0 < BN; c0 += cols_per_store) {
        if (n0 + c0 >= args.n || !rows_live) break;  // fully clipped: nothing to store
        const int sbuf = store_idx & 1;
        // The store issued two steps ago read from this staging buffer.
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        uint8_t* row = stage_buf + sbuf * EPI_BUF_BYTES + lane * 128;
        const int sw = lane & 7;
        if (args.out_f32) {
          uint32_t v[32];
          tc_ld_32x32(t_row + c0, v);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 o;
            o.x = __uint_as_float(v[4 * j + 0]);
            o.y = __uint_as_float(v[4 * j + 1]);
            o.z = __uint_as_float(v[4 * j + 2]);
            o.w = __uint_as_float(v[4 * j + 3]);
            if (args.relu) {
              o.x = fmaxf(o.x, 0.f); o.y = fmaxf(o.y, 0.f);
              o.z = fmaxf(o.z, 0.f); o.w = fmaxf(o.w, 0.f);
            }
            *reinterpret_cast<float4*>(row + ((j ^ sw) << 4)) = o;
          }
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t v[32];
            tc_ld_32x32(t_row + c0 + h * 32, v);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                f[e] = __uint_as_float(v[8 * j + e]);
                if (args.relu) f[e] = fmaxf(f[e], 0.f);
              }
              uint4 o;
              o.x = pack_bf16x2(f[0], f[1]);
              o.y = pack_bf16x2(f[2], f[3]);
              o.z = pack_bf16x2(f[4], f[5]);
              o.w = pack_bf16x2(f[6], f[7]);
              *reinterpret_cast<uint4*>(row + (((h * 4 + j) ^ sw) << 4)) = o;
            }
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(&map_c, stage_u32 + sbuf * EPI_BUF_BYTES, n0 + c0, m0 + q * 32, b);
          tma_store_commit();
        }
        ++store_idx;
      }
      // All tcgen05.ld of this accumulator have completed (wait::ld above).
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty_bar(buf));
    }
    if (lane == 0) tma_store_wait_all();
    if (!ok && lane == 0 && args.status) atomicExch(args.status, MTFC_ERR_TIMEOUT);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// ------------------------------------------------- the 2-CTA (cta_group::2) kernel
// A cluster of two CTAs on neighbouring SMs computes one 256x256 tile: CTA r
// holds rows [128r, 128r+128) of A and columns [128r, 128r+128) of B for each
// K block, the leader (rank 0) issues tcgen05.mma.cta_group::2 128x256 per SM
// reading both CTAs' shared memory, and each CTA's TMEM receives its 128 rows
// of the accumulator.  B crosses L2->SM once per pair instead of once per SM
// and each SM's shared memory serves 64 B/clk of operand reads instead of 96,
// which is what lifts the single-CTA kernel's shared-memory bandwidth ceiling.
// No load uses multicast: each CTA fetches its own halves with plain TMA loads
// that report to the leader's mbarrier.
constexpr int B2_STAGE_BYTES = (BN / 2) * BK * 2;  // 16 KiB: this CTA's half of B
// Shared-memory plan of the pair kernel.  The fused GEMM+allreduce variant trades
// one pipeline stage for two more staging buffers per epilogue warp: half of its
// output tiles are stored into a peer GPU's memory, and such a store holds its
// staging buffer for a NVLink round trip.
template <bool FUSED>
struct PairCfg {
  static constexpr int STAGES = FUSED ? 5 : 6;
  static constexpr int EPI_BUFS = FUSED ? 4 : 2;  // staging buffers per epilogue warp
  static constexpr int A = 0;
  static constexpr int B = A + STAGES * A_STAGE_BYTES;
  static constexpr int EPI = B + STAGES * B2_STAGE_BYTES;
  static constexpr int BAR = EPI + EPI_WARPS * EPI_BUFS * EPI_BUF_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4;
  static constexpr int MISC = BAR + NUM_BARS * 8;
  static constexpr int USED = MISC + 16;
  static constexpr int ALLOC = USED + 1024;
};
constexpr int SMEM2_ALLOC = PairCfg<false>::ALLOC;
constexpr int SMEM2F_ALLOC = PairCfg<true>::ALLOC;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// shared::cluster address of `addr` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}

// TMA load whose completion bytes are reported to an mbarrier that may live in
// the peer CTA of the pair (cluster address), data landing in this CTA.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map,
                                                 uint32_t bar_cluster_addr, int c0, int c1,
                                                 int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1),
        "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar_cluster_addr)
               : "memory");
}

__device__ __forceinline__ void tc_mma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ------------------------------------------------ GEMM fused with its allreduce
// The same pair kernel with the SUM allreduce of its output over `nranks` GPUs
// (one process each) folded in.  Row blocks of 256 output rows are owned
// round-robin (block rb by rank rb % nranks).  The epilogue of every rank stores
// its partial tile straight into the OWNER's staging buffer (a TMA store into
// peer memory: slot [source rank][k-th owned block]), so the reduce-scatter half
// of the exchange rides on stores the epilogue issues anyway.  Every CTA carries
// four extra "comm" warps that take no part in the product: once all ranks have
// delivered a row block this rank owns, the comm warps of one CTA add the nranks
// partial copies of a slice of it (local reads; see reduce_block for the
// arithmetic) and write the sum into every rank's output buffer (plain 16-byte
// stores, local and peer).  The loop is bound by memory latency, so spreading it
// over all SMs (beside the MMA pipeline, which leaves the load/store units idle)
// buys the bytes in flight that a few dedicated CTAs cannot have.  Clusters walk
// the tiles row block by row block, so block i is exchanged while the blocks
// after it are still being multiplied.
//
// Flags (uint32, in peer-visible memory, never reset; a launch compares against
// epoch * count): flags[rb] on the owner of row block rb counts epilogue warps
// of all ranks that have delivered their part of rb; flags[FLAG_DONE] on every
// rank counts row-block slices written into that rank's output.  `ctl` is this rank's
// private triple {launches completed, CTAs whose comm warps finished in this launch,
// next slice to hand out}; keeping
// the epoch on the device lets a captured launch be replayed.  Every wait is
// bounded: a rank whose peers never show up raises MTFC_ERR_TIMEOUT in the status
// word and returns.
constexpr int MAX_RANKS = 8;
constexpr int FLAG_DONE = 4096;  // row-block counters live in [0, FLAG_DONE)
constexpr int COMM_UNROLL = 8;   // 16-byte vectors per thread in flight, general rank count
constexpr int COMM_LOADS = 32;   // 16-byte loads per thread in flight for 2, 4 or 8 ranks
constexpr long long PEER_WAIT_CYCLES_DEFAULT = 6000000000LL;  // ~3 s
constexpr int COMM_UNIT_ROWS = 32;
constexpr int COMM_WARPS = 4;
constexpr int COMM_THREADS = 32 * COMM_WARPS;
constexpr int NUM_THREADS_FUSED = NUM_THREADS + COMM_THREADS;

struct FusedArgs {
  CUtensorMap stage_map[MAX_RANKS];  // rank o's staging buffer [nranks * blocks_per_rank * 256, n]
  const uint8_t* stage;              // this rank's staging buffer
  uint8_t* out[MAX_RANKS];
  uint32_t* flags[MAX_RANKS];
  uint32_t* ctl;
  int rank, nranks;
  int blocks_per_rank;
  long long wait_cycles;  // how long a wait for another rank may last
  // Exchange form.
  //   EXCHANGE_PUSH: the epilogue stores each partial tile into the owner's staging
  //     buffer (remote TMA stores); the owner adds local copies.
  //   EXCHANGE_PULL: every rank keeps its partial product in its OWN staging buffer at
  //     the output's row offsets (part_map), so the epilogue never waits on NVLink; the
  //     owner's comm warps read the other ranks' copies with plain peer loads.
  //   EXCHANGE_MULTIMEM: partial products local as for PULL; the owner reads the SUM of
  //     all ranks' copies through the staging buffers' multicast address
  //     (multimem.ld_reduce: NVSwitch adds the copies in fp32) and writes it to all ranks'
  //     outputs through the output buffers' multicast address (multimem.st).
  int exchange;
  const uint8_t* stage_all[MAX_RANKS];
  const uint8_t* mc_stage;
  uint8_t* mc_out;
  CUtensorMap part_map;
};
constexpr int EXCHANGE_PUSH = 0;
constexpr int EXCHANGE_PULL = 1;
constexpr int EXCHANGE_MULTIMEM = 2;

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Waits (bounded) until *p has reached `target` (wrap-safe comparison).
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* p, uint32_t target, long long limit) {
  const long long t0 = clock64();
  for (;;) {
    if ((int32_t)(ld_acquire_sys(p) - target) >= 0) return true;
    if (clock64() - t0 > limit) return false;
    __nanosleep(128);
  }
}
// 16-byte load served from L2, which never hits a stale L1 line (the data was written by TMA
// stores of other SMs and other GPUs during this launch).
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// cp.async.bulk.wait_group with a run-time count: returns once at most `pending`
// of this thread's newest bulk groups are still incomplete (0..8).
__device__ __forceinline__ void bulk_wait_upto(int pending) {
  switch (pending) {
    case 0: asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.bulk.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.bulk.wait_group 2;" ::: "memory"); break;
    case 3: asm volatile("cp.async.bulk.wait_group 3;" ::: "memory"); break;
    case 4: asm volatile("cp.async.bulk.wait_group 4;" ::: "memory"); break;
    case 5: asm volatile("cp.async.bulk.wait_group 5;" ::: "memory"); break;
    case 6: asm volatile("cp.async.bulk.wait_group 6;" ::: "memory"); break;
    case 7: asm volatile("cp.async.bulk.wait_group 7;" ::: "memory"); break;
    default: asm volatile("cp.async.bulk.wait_group 8;" ::: "memory"); break;
  }
}
__device__ __forceinline__ void st_v4(void* p, const uint4& v) {
  asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// acc += the eight bf16 values of x, widened exactly to fp32.
__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& x) {
  const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    acc[2 * e] += __uint_as_float(w[e] << 16);
    acc[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
  }
}

__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint4 add_bf16x8_packed(const uint4& a, const uint4& b) {
  return make_uint4(add_bf16x2(a.x, b.x), add_bf16x2(a.y, b.y), add_bf16x2(a.z, b.z),
                    add_bf16x2(a.w, b.w));
}

// Sum of the n copies of part of a row block (src[s], s < n; local or peer memory),
// nvec 16-byte vectors, written to every rank's output at out_off.
// NR = n when n is 2, 4 or 8: the loads of all copies of COMM_LOADS / NR vectors
// are in flight together, and the sum is a balanced tree of packed bf16 additions
// (for two ranks that is the correctly rounded sum; for four and eight, log2(n)
// roundings, where a ring allreduce in bf16 has n - 1): four instructions per
// 16 bytes and level, so that the warps doing this beside the MMA pipeline take
// few issue slots.  NR = 1 is the general form: one copy at a time, accumulated
// in fp32 and rounded once.
template <int NR>
__device__ __forceinline__ void reduce_block(const uint8_t* const* src, uint8_t* const* out,
                                             long long out_off, long long nvec, int n, int tid) {
  constexpr int U = NR == 1 ? COMM_UNROLL : COMM_LOADS / NR;
  for (long long v0 = tid; v0 < nvec; v0 += (long long)COMM_THREADS * U) {
    uint4 res[U];
    if (NR == 1) {
      float acc[U][8];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
      for (int s = 0; s < n; ++s) {
        uint4 x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long v = v0 + (long long)u * COMM_THREADS;
          x[u] = v < nvec ? ld_cg_v4(src[s] + v * 16) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) add_bf16x8(acc[u], x[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        res[u].x = pack_bf16x2(acc[u][0], acc[u][1]);
        res[u].y = pack_bf16x2(acc[u][2], acc[u][3]);
        res[u].z = pack_bf16x2(acc[u][4], acc[u][5]);
        res[u].w = pack_bf16x2(acc[u][6], acc[u][7]);
      }
    } else {
      uint4 x[NR][U];
#pragma unroll
      for (int s = 0; s < NR; ++s)
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const long long v = v0 + (long long)u * COMM_THREADS;
          x[s][u] = v < nvec ? ld_cg_v4(src[s] + v * 16) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
      for (int width = NR / 2; width >= 1; width /= 2)   // ranks (0+1)+(2+3) ..., the same on every owner
#pragma unroll
        for (int s = 0; s < width; ++s)
#pragma unroll
          for (int u = 0; u < U; ++u) x[s][u] = add_bf16x8_packed(x[2 * s][u], x[2 * s + 1][u]);
#pragma unroll
      for (int u = 0; u < U; ++u) res[u] = x[0][u];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long v = v0 + (long long)u * COMM_THREADS;
      if (v < nvec)
        for (int p = 0; p < n; ++p) st_v4(out[p] + out_off + v * 16, res[u]);
    }
  }
}

// Sum over all ranks of eight bf16 values at a multicast address, accumulated in fp32
// inside the switch and rounded once.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
// 16 bytes to the same offset of every rank's buffer.
__device__ __forceinline__ void multimem_st_v4(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}

// The switch-reduced form of reduce_block: nvec 16-byte vectors starting at byte
// offset `off` of the (symmetric) staging and output buffers.
__device__ __forceinline__ void reduce_block_multimem(const uint8_t* mc_src, uint8_t* mc_dst,
                                                      long long off, long long nvec, int tid) {
  constexpr int U = COMM_UNROLL;
  for (long long v0 = tid; v0 < nvec; v0 += (long long)COMM_THREADS * U) {
    uint4 x[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long v = v0 + (long long)u * COMM_THREADS;
      if (v < nvec) x[u] = multimem_ld_reduce_bf16x8(mc_src + off + v * 16);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long v = v0 + (long long)u * COMM_THREADS;
      if (v < nvec) multimem_st_v4(mc_dst + off + v * 16, x[u]);
    }
  }
}

__device__ __forceinline__ void comm_warps_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(COMM_THREADS) : "memory");
}

// The comm warps of one CTA (threads NUM_THREADS ..).  Work units are slices of
// COMM_UNIT_ROWS rows of the row blocks this rank owns, numbered in the order the
// blocks complete and claimed one at a time from a counter (ctl[2]): whichever
// CTA is free takes the next slice, so the slices of the last blocks - the only
// ones not hidden behind the product - spread over all SMs.
__device__ void allreduce_comm_warps(uint8_t* smem, const GemmArgs& args, const FusedArgs& fa) {
  const int n = fa.nranks;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + PairCfg<true>::MISC + 12);
  volatile uint32_t* word = reinterpret_cast<volatile uint32_t*>(smem + PairCfg<true>::MISC + 8);
  const int tid = (int)threadIdx.x - NUM_THREADS;
  if (tid == 0) {
    *abort_flag = 0;
    *word = ld_acquire_sys(fa.ctl) + 1u;
  }
  comm_warps_sync();
  const uint32_t epoch = *word;
  comm_warps_sync();
  constexpr int UNITS = 2 * BM / COMM_UNIT_ROWS;  // per row block
  const long long row_bytes = (long long)args.n * 2;
  const long long block_bytes = 2LL * BM * row_bytes;
  const int num_rb = args.tiles_m;
  const int owned = num_rb > fa.rank ? (num_rb - fa.rank + n - 1) / n : 0;
  const uint32_t ready_target = epoch * (uint32_t)(n * args.tiles_n * 2 * EPI_WARPS);
  bool ok = true;
  for (;;) {
    if (tid == 0) *word = atomicAdd(fa.ctl + 2, 1u);
    comm_warps_sync();
    const int w = (int)*word;
    comm_warps_sync();
    if (w >= UNITS * owned) break;
    const int k = w / UNITS, sub = w % UNITS;
    const int rb = fa.rank + n * k;
    if (tid == 0 && !wait_flag_ge(fa.flags[fa.rank] + rb, ready_target, fa.wait_cycles)) *abort_flag = 1;
    comm_warps_sync();
    if (*abort_flag) { ok = false; break; }
    const int rows = max(0, min(COMM_UNIT_ROWS, args.m - rb * 2 * BM - sub * COMM_UNIT_ROWS));
    const long long nvec = (rows * row_bytes) >> 4;
    const long long sub_off = (long long)sub * COMM_UNIT_ROWS * row_bytes;
    const long long out_off = (long long)rb * block_bytes + sub_off;
    if (fa.exchange == EXCHANGE_MULTIMEM) {
      reduce_block_multimem(fa.mc_stage, fa.mc_out, out_off, nvec, tid);
    } else {
      const uint8_t* src[MAX_RANKS];
      if (fa.exchange == EXCHANGE_PULL) {
        // rank s's partial of this row block sits in ITS staging buffer at the output's offset
        for (int s = 0; s < n; ++s) src[s] = fa.stage_all[s] + out_off;
      } else {
        // all ranks' partials were stored into this rank's staging buffer, slot [source][k]
        const long long src_stride = (long long)fa.blocks_per_rank * block_bytes;
        for (int s = 0; s < n; ++s) src[s] = fa.stage + (long long)k * block_bytes + sub_off + s * src_stride;
      }
      switch (n) {
        case 2: reduce_block<2>(src, fa.out, out_off, nvec, n, tid); break;
        case 4: reduce_block<4>(src, fa.out, out_off, nvec, n, tid); break;
        case 8: reduce_block<8>(src, fa.out, out_off, nvec, n, tid); break;
        default: reduce_block<1>(src, fa.out, out_off, nvec, n, tid); break;
      }
    }
    // the barrier orders every thread's stores before thread 0's release, which
    // is cumulative: one system-scope release per slice, no separate fence
    comm_warps_sync();
    if (tid == 0) {
      for (int p = 0; p < n; ++p) red_release_sys_add(fa.flags[p] + FLAG_DONE, 1u);
    }
  }
  if (tid == 0) {
    if (!ok) {
      if (args.status) atomicExch(args.status, MTFC_ERR_TIMEOUT);
    } else if (atomicAdd(fa.ctl + 1, 1u) == gridDim.x - 1) {
      // last CTA of this launch: the output is whole once every half row block
      // has been written here, and only then may the next launch start
      if (wait_flag_ge(fa.flags[fa.rank] + FLAG_DONE, epoch * (uint32_t)(UNITS * num_rb),
                       fa.wait_cycles)) {
        fa.ctl[1] = 0u;
        fa.ctl[2] = 0u;
        __threadfence();
        fa.ctl[0] = epoch;
      } else if (args.status) {
        atomicExch(args.status, MTFC_ERR_TIMEOUT);
      }
    }
  }
}


__device__ __forceinline__ uint32_t make_idesc_pair(int a_mn, int b_mn) {
  uint32_t d = 0;
  d |= 1u << 4;
  d |= 1u << 7;
  d |= 1u << 10;
  d |= (uint32_t)(a_mn & 1) << 15;
  d |= (uint32_t)(b_mn & 1) << 16;
  d |= (uint32_t)(BN >> 3) << 17;
  d |= (uint32_t)((2 * BM) >> 4) << 24;  // M = 256 across the pair
  return d;
}

template <bool FUSED>
__device__ __forceinline__ void pair_gemm_body(const CUtensorMap& map_a, const CUtensorMap& map_b,
                                               const CUtensorMap& map_c, const GemmArgs& args,
                                               const FusedArgs* fa) {
  using Cfg = PairCfg<FUSED>;
  constexpr int STAGES2 = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_base + Cfg::BAR;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES2 + s); };
  auto tmem_full_bar = [&](int b) { return bar_base + 8u * (2 * STAGES2 + b); };
  auto tmem_empty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES2 + 2 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Cfg::MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Cfg::MISC + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(full_bar(s), 1);   // leader's: its producer's expect_tx arrival
      mbar_init(empty_bar(s), 1);  // one tcgen05.commit per use, in each CTA
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tmem_full_bar(b), 1);
      mbar_init(tmem_empty_bar(b), 2 * EPI_WARPS);  // leader's: epilogue warps of both CTAs
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_base + Cfg::MISC),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_kb = (args.k + BK - 1) / BK;
  const long long tiles_per_batch = (long long)args.tiles_m * args.tiles_n;  // 256x256 tiles
  const long long num_tiles = tiles_per_batch * args.batch;
  const long long cluster_id = blockIdx.x >> 1;
  const long long num_clusters = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (long long t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        const int b = (int)(t / tiles_per_batch);
        const int r = (int)(t % tiles_per_batch);
        const int m0 = (r / args.tiles_n) * (2 * BM) + (int)rank * BM;
        const int n0 = (r % args.tiles_n) * BN + (int)rank * (BN / 2);
        const int ab = args.a_batched ? b : 0;
        const int bb = args.b_batched ? b : 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) { ok = false; break; }
          if (leader) mbar_expect_tx(full_bar(stage), 2 * (A_STAGE_BYTES + B2_STAGE_BYTES));
          const uint32_t lead_full = map_to_cta(full_bar(stage), 0);
          const uint32_t sa = smem_base + Cfg::A + stage * A_STAGE_BYTES;
          const uint32_t sb = smem_base + Cfg::B + stage * B2_STAGE_BYTES;
          const int k0 = kb * BK;
          if (args.a_mn_major) {
#pragma unroll
            for (int g = 0; g < BM / 64; ++g)
              tma_load_3d_pair(sa + g * MN_GROUP_BYTES, &map_a, lead_full, m0 + g * 64, k0, ab);
          } else {
            tma_load_3d_pair(sa, &map_a, lead_full, k0, m0, ab);
          }
          if (args.b_mn_major) {
#pragma unroll
            for (int g = 0; g < BN / 128; ++g)
              tma_load_3d_pair(sb + g * MN_GROUP_BYTES, &map_b, lead_full, n0 + g * 64, k0, bb);
          } else {
            tma_load_3d_pair(sb, &map_b, lead_full, k0, n0, bb);
          }
          if (++stage == STAGES2) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok && args.status) atomicExch(args.status, MTFC_ERR_TIMEOUT);
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && leader) {
      const uint32_t idesc = make_idesc_pair(args.a_mn_major, args.b_mn_major);
      const uint32_t a_lbo = args.a_mn_major ? MN_GROUP_BYTES : 16;
      const uint32_t b_lbo = args.b_mn_major ? MN_GROUP_BYTES : 16;
      const uint32_t a_kstep = args.a_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_kstep = args.b_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long local = 0;
      for (long long t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local) {
        const int buf = (int)(local & 1);
        const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
        if (!mbar_wait(tmem_empty_bar(buf), acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + Cfg::A + stage * A_STAGE_BYTES;
          const uint32_t sb = smem_base + Cfg::B + stage * B2_STAGE_BYTES;
#pragma unroll
          for (int ks = 0; ks < BK / UMMA_K; ++ks) {
            const uint64_t da = make_smem_desc(sa + ks * a_kstep, a_lbo, 1024);
            const uint64_t db = make_smem_desc(sb + ks * b_kstep, b_lbo, 1024);
            tc_mma_bf16_pair(d_tmem, da, db, idesc, (kb | ks) != 0 ? 1u : 0u);
          }
          // free the stage in both CTAs once these MMAs have read it
          tc_commit_pair(map_to_cta(empty_bar(stage), 0));
          tc_commit_pair(map_to_cta(empty_bar(stage), 1));
          if (++stage == STAGES2) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit_pair(map_to_cta(tmem_full_bar(buf), 0));
        tc_commit_pair(map_to_cta(tmem_full_bar(buf), 1));
      }
      if (!ok && args.status) atomicExch(args.status, MTFC_ERR_TIMEOUT);
    }
  } else if (FUSED && warp >= 2 + EPI_WARPS) {
    // ------------------------------------------------ comm warps (fused kernel only)
    allreduce_comm_warps(smem, args, *fa);
  } else {
    // ------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    const int ew = warp - 2;
    uint8_t* stage_buf = smem + Cfg::EPI + ew * Cfg::EPI_BUFS * EPI_BUF_BYTES;
    const uint32_t stage_u32 = smem_base + Cfg::EPI + ew * Cfg::EPI_BUFS * EPI_BUF_BYTES;
    const int cols_per_store = args.out_f32 ? 32 : 64;
    bool ok = true;
    long long local = 0;
    int store_idx = 0;
    // fused: row blocks of the last two tiles, whose arrival is not yet signalled, and
    // the number of store groups of the newer one
    int pending_rb = -1, older_rb = -1, pending_stores = 0;
    for (long long t = cluster_id; t < num_tiles && ok; t += num_clusters, ++local) {
      const int tile_first_store = store_idx;
      const int buf = (int)(local & 1);
      const uint32_t acc_phase = (uint32_t)((local >> 1) & 1);
      const int b = (int)(t / tiles_per_batch);
      const int r = (int)(t % tiles_per_batch);
      const int m0 = (r / args.tiles_n) * (2 * BM) + (int)rank * BM;
      const int n0 = (r % args.tiles_n) * BN;
      // fused: the tile goes to the staging buffer of its row block's owner
      const int rb = r / args.tiles_n;
      const CUtensorMap* dst_map = &map_c;
      int dst_row = m0 + q * 32;
      if (FUSED) {
        if (fa->exchange != EXCHANGE_PUSH) {
          dst_map = &fa->part_map;   // own staging buffer, at the output's row offsets
        } else {
          dst_map = &fa->stage_map[rb % fa->nranks];
          dst_row = (fa->rank * fa->blocks_per_rank + rb / fa->nranks) * (2 * BM) + (int)rank * BM + q * 32;
        }
      }
      ok = __all_sync(0xffffffffu, mbar_wait(tmem_full_bar(buf), acc_phase, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
      const bool rows_live = (m0 + q * 32) < args.m;
      for (int c0 = 0; c0 < BN; c0 += cols_per_store) {
        if (n0 + c0 >= args.n || !rows_live) break;
        const int sbuf = store_idx % Cfg::EPI_BUFS;
        if (lane == 0) tma_store_wait_read<Cfg::EPI_BUFS - 1>();
        __syncwarp();
        uint8_t* row = stage_buf + sbuf * EPI_BUF_BYTES + lane * 128;
        const int sw = lane & 7;
        if (args.out_f32) {
          uint32_t v[32];
          tc_ld_32x32(t_row + c0, v);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 o;
            o.x = __uint_as_float(v[4 * j + 0]);
            o.y = __uint_as_float(v[4 * j + 1]);
            o.z = __uint_as_float(v[4 * j + 2]);
            o.w = __uint_as_float(v[4 * j + 3]);
            if (args.relu) {
              o.x = fmaxf(o.x, 0.f); o.y = fmaxf(o.y, 0.f);
              o.z = fmaxf(o.z, 0.f); o.w = fmaxf(o.w, 0.f);
            }
            *reinterpret_cast<float4*>(row + ((j ^ sw) << 4)) = o;
          }
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t v[32];
            tc_ld_32x32(t_row + c0 + h * 32, v);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                f[e] = __uint_as_float(v[8 * j + e]);
                if (args.relu) f[e] = fmaxf(f[e], 0.f);
              }
              uint4 o;
              o.x = pack_bf16x2(f[0], f[1]);
              o.y = pack_bf16x2(f[2], f[3]);
              o.z = pack_bf16x2(f[4], f[5]);
              o.w = pack_bf16x2(f[6], f[7]);
              *reinterpret_cast<uint4*>(row + (((h * 4 + j) ^ sw) << 4)) = o;
            }
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(dst_map, stage_u32 + sbuf * EPI_BUF_BYTES, n0 + c0, dst_row, b);
          tma_store_commit();
        }
        ++store_idx;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tmem_empty_bar(buf), 0));
      if ((FUSED || args.progress) && lane == 0) {
        // Tell the owner of the row block of the tile TWO tiles back that this
        // warp's part of it has arrived (complete, not merely read out of the
        // staging buffers): its stores have had two tile times to land, so the
        // wait for "all but the store groups of the last two tiles" returns at
        // once, where waiting for this tile's own stores would stall the epilogue
        // for a round trip over NVLink per tile.
        const int mine = store_idx - tile_first_store;
        if (older_rb >= 0) {
          bulk_wait_upto(mine + pending_stores);
          red_release_sys_add(FUSED ? fa->flags[older_rb % fa->nranks] + older_rb
                                    : args.progress + older_rb, 1u);
        }
        older_rb = pending_rb;
        pending_rb = rb;
        pending_stores = mine;
      }
    }
    if (lane == 0) tma_store_wait_all();
    if ((FUSED || args.progress) && lane == 0) {
      if (older_rb >= 0)
        red_release_sys_add(FUSED ? fa->flags[older_rb % fa->nranks] + older_rb : args.progress + older_rb, 1u);
      if (pending_rb >= 0)
        red_release_sys_add(FUSED ? fa->flags[pending_rb % fa->nranks] + pending_rb
                                  : args.progress + pending_rb, 1u);
    }
    if (!ok && lane == 0 && args.status) atomicExch(args.status, MTFC_ERR_TIMEOUT);
  }

  // Neither CTA may leave while the pair's MMAs can still read its shared memory.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
einsum_gemm_tcgen05_2cta(const __grid_constant__ CUtensorMap map_a,
                         const __grid_constant__ CUtensorMap map_b,
                         const __grid_constant__ CUtensorMap map_c, const GemmArgs args) {
  pair_gemm_body<false>(map_a, map_b, map_c, args, nullptr);
}

__global__ void __launch_bounds__(NUM_THREADS_FUSED, 1)
einsum_gemm_allreduce_2cta(const __grid_constant__ CUtensorMap map_a,
                           const __grid_constant__ CUtensorMap map_b, const GemmArgs args,
                           const __grid_constant__ FusedArgs fa) {
  pair_gemm_body<true>(map_a, map_b, fa.stage_map[0], args, &fa);
}

// ------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

// 3-D map {inner, outer, batch} with a {box_inner, box_outer, 1} box, 128B swizzle.
int encode_map(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base,
               int64_t inner, int64_t outer, int64_t batch, int64_t outer_stride,
               int64_t batch_stride, int box_inner, int box_outer, const char* what) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(MTFC_ERR_CUDA, "cuTensorMapEncodeTiled entry point unavailable");
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)batch};
  // Strides of extent-1 dims are never used for addressing but must still be
  // valid (non-zero multiples of 16 bytes).
  int64_t os = outer_stride * elem_bytes;
  if (outer == 1 || os <= 0) os = ((inner * elem_bytes + 15) / 16) * 16;
  int64_t bs = batch_stride * elem_bytes;
  if (batch == 1 || bs <= 0) bs = os * outer;
  cuuint64_t strides[2] = {(cuuint64_t)os, (cuuint64_t)bs};
  cuuint32_t box[3] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(MTFC_ERR_SHAPE,
                "tensor map for %s rejected (CUresult %d): inner=%lld outer=%lld batch=%lld "
                "strides=%lld,%lld B",
                what, (int)r, (long long)inner, (long long)outer, (long long)batch, (long long)os,
                (long long)bs);
  return MTFC_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Operand layout classification: 0 = K-major, 1 = MN-major, -1 = not TMA-able.
int classify(int64_t mn, int64_t k, int64_t s_mn, int64_t s_k, int64_t batch, int64_t s_batch) {
  if (batch > 1 && (s_batch % 8 != 0 || s_batch <= 0)) return -1;
  if ((s_k == 1 || k == 1) && (mn == 1 || (s_mn % 8 == 0 && s_mn >= k))) return 0;
  if ((s_mn == 1 || mn == 1) && (k == 1 || (s_k % 8 == 0 && s_k >= mn))) return 1;
  return -1;
}

}  // namespace

bool gemm_tcgen05_eligible(const mtfc_gemm_desc* d, const void* a, const void* b, const void* c) {
  if (d->in_dtype != MTFC_BF16) return false;
  if (d->out_dtype != MTFC_BF16 && d->out_dtype != MTFC_F32) return false;
  if (d->batch < 1 || d->m < 1 || d->n < 1 || d->k < 1) return false;
  if (d->m > INT32_MAX || d->n > INT32_MAX || d->k > INT32_MAX || d->batch > INT32_MAX)
    return false;
  if (!aligned16(a) || !aligned16(b) || !aligned16(c)) return false;
  const bool a_b = d->batch > 1 && d->a_batch != 0;
  const bool b_b = d->batch > 1 && d->b_batch != 0;
  if (classify(d->m, d->k, d->a_m, d->a_k, a_b ? d->batch : 1, d->a_batch) < 0) return false;
  if (classify(d->n, d->k, d->b_n, d->b_k, b_b ? d->batch : 1, d->b_batch) < 0) return false;
  const int64_t oe = d->out_dtype == MTFC_F32 ? 4 : 2;
  if (d->n > 1 && d->c_n != 1) return false;
  if (d->m > 1 && ((d->c_m * oe) % 16 != 0 || d->c_m < d->n)) return false;
  if (d->batch > 1 && ((d->c_batch * oe) % 16 != 0 || d->c_batch <= 0)) return false;
  return true;
}

// Resident 2-CTA clusters the device can hold for the pair kernel (0 if the
// query fails); cached per device.
int max_pair_clusters() {
  static int cached[64];
  static bool known[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!known[dev]) {
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (unsigned)sm_count(), 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM2_ALLOC;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaFuncSetAttribute(einsum_gemm_tcgen05_2cta, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM2_ALLOC) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, einsum_gemm_tcgen05_2cta, &cfg) != cudaSuccess)
      n = 0;
    (void)cudaGetLastError();
    cached[dev] = n;
    known[dev] = true;
  }
  return cached[dev];
}

// cta_group: 0 = choose, 1 = single-CTA kernel, 2 = CTA-pair kernel.
int gemm_tcgen05_launch(const mtfc_gemm_desc* d, const void* a, const void* b, void* c,
                        cudaStream_t stream, int cta_group, void* progress) {
  int pair_clusters = 0;
  if (cta_group != 1) pair_clusters = max_pair_clusters();
  // The pair kernel works on 256-row tiles: worth it once M fills them.
  bool use_pair = pair_clusters > 0 && (cta_group == 2 || d->m >= 256);
  if (cta_group == 2 && pair_clusters <= 0)
    return fail(MTFC_ERR_CUDA, "CTA-pair GEMM forced but no 2-CTA cluster can be resident");
  const bool a_b = d->batch > 1 && d->a_batch != 0;
  const bool b_b = d->batch > 1 && d->b_batch != 0;
  const int a_major = classify(d->m, d->k, d->a_m, d->a_k, a_b ? d->batch : 1, d->a_batch);
  const int b_major = classify(d->n, d->k, d->b_n, d->b_k, b_b ? d->batch : 1, d->b_batch);
  if (a_major < 0 || b_major < 0) return fail(MTFC_ERR_SHAPE, "operand layout not TMA-able");

  CUtensorMap map_a, map_b, map_c;
  int rc;
  if (a_major == 0)
    rc = encode_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, d->k, d->m,
                    a_b ? d->batch : 1, d->a_m, d->a_batch, BK, BM, "A (K-major)");
  else
    rc = encode_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, d->m, d->k,
                    a_b ? d->batch : 1, d->a_k, d->a_batch, 64, BK, "A (M-major)");
  if (rc != MTFC_OK) return rc;
  if (b_major == 0)
    rc = encode_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b, d->k, d->n,
                    b_b ? d->batch : 1, d->b_n, d->b_batch, BK, use_pair ? BN / 2 : BN,
                    "B (K-major)");
  else
    rc = encode_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b, d->n, d->k,
                    b_b ? d->batch : 1, d->b_k, d->b_batch, 64, BK, "B (N-major)");
  if (rc != MTFC_OK) return rc;
  const bool out_f32 = d->out_dtype == MTFC_F32;
  rc = encode_map(&map_c, out_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                  out_f32 ? 4 : 2, c, d->n, d->m, d->batch, d->c_m, d->c_batch, out_f32 ? 32 : 64,
                  32, "C");
  if (rc != MTFC_OK) return rc;

  GemmArgs args;
  args.m = (int)d->m;
  args.n = (int)d->n;
  args.k = (int)d->k;
  args.batch = (int)d->batch;
  const int tile_rows = use_pair ? 2 * BM : BM;
  args.tiles_m = (int)((d->m + tile_rows - 1) / tile_rows);
  args.tiles_n = (int)((d->n + BN - 1) / BN);
  args.a_mn_major = a_major;
  args.b_mn_major = b_major;
  args.a_batched = a_b ? 1 : 0;
  args.b_batched = b_b ? 1 : 0;
  args.relu = d->epilogue == MTFC_EPILOGUE_RELU;
  args.out_f32 = out_f32 ? 1 : 0;
  args.status = device_status_word();
  args.progress = static_cast<uint32_t*>(progress);
  if (progress && !(use_pair && d->batch == 1))
    return fail(MTFC_ERR_UNSUPPORTED, "gemm: progress counters need the CTA-pair kernel and batch 1");

  const long long num_tiles = (long long)args.tiles_m * args.tiles_n * args.batch;
  if (use_pair) {
    const long long clusters = num_tiles < pair_clusters ? num_tiles : pair_clusters;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM2_ALLOC;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MTFC_CUDA(cudaLaunchKernelEx(&cfg, einsum_gemm_tcgen05_2cta, map_a, map_b, map_c, args));
    return MTFC_OK;
  }

  static bool attr_set[64] = {false};
  int dev = 0;
  MTFC_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    MTFC_CUDA(cudaFuncSetAttribute(einsum_gemm_tcgen05, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   SMEM_ALLOC));
    attr_set[dev] = true;
  }
  const int sms = sm_count();
  const unsigned grid = (unsigned)(num_tiles < sms ? num_tiles : sms);
  einsum_gemm_tcgen05<<<grid, NUM_THREADS, SMEM_ALLOC, stream>>>(map_a, map_b, map_c, args);
  MTFC_LAUNCH_CHECK("einsum_gemm_tcgen05");
  return MTFC_OK;
}

int gemm_allreduce_flag_bytes() { return (FLAG_DONE + 1) * 4; }

static long long g_peer_wait_cycles = PEER_WAIT_CYCLES_DEFAULT;
static int g_cooperative_ok = 1, g_cooperative_launched = 0;

// Limit of every wait on another rank inside the fused kernel, in milliseconds
// at a nominal 2 GHz clock; <= 0 restores the default of about 3 s.
void gemm_allreduce_set_wait_ms(int ms) {
  g_peer_wait_cycles = ms > 0 ? (long long)ms * 2000000LL : PEER_WAIT_CYCLES_DEFAULT;
}

// Resident 2-CTA clusters for the fused kernel (its blocks are larger); cached per device.
int max_fused_clusters() {
  static int cached[64];
  static bool known[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!known[dev]) {
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (unsigned)sm_count(), 1, 1);
    cfg.blockDim = dim3(NUM_THREADS_FUSED, 1, 1);
    cfg.dynamicSmemBytes = SMEM2F_ALLOC;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaFuncSetAttribute(einsum_gemm_allreduce_2cta, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SMEM2F_ALLOC) != cudaSuccess ||
        cudaOccupancyMaxActiveClusters(&n, einsum_gemm_allreduce_2cta, &cfg) != cudaSuccess)
      n = 0;
    (void)cudaGetLastError();
    cached[dev] = n;
    known[dev] = true;
  }
  return cached[dev];
}

long long gemm_allreduce_stage_bytes(long long m, long long n, int nranks) {
  if (m < 1 || n < 1 || nranks < 1) return 0;
  const long long num_rb = (m + 2 * BM - 1) / (2 * BM);
  const long long bpr = (num_rb + nranks - 1) / nranks;
  return (long long)nranks * bpr * 2 * BM * n * 2;
}

// GEMM with the allreduce of its bf16 [m, n] row-major output folded in (see
// the kernel comment).  `stage`, `out` and `flags` hold every rank's buffer
// address as seen from this process; `ctl` is this rank's private 16 bytes.
int gemm_allreduce_launch(const mtfc_gemm_desc* d, const void* a, const void* b,
                          void* const* stage, void* const* out, void* const* flags, void* ctl,
                          int rank, int nranks, int exchange, const void* mc_stage, void* mc_out,
                          cudaStream_t stream) {
  if (nranks < 2 || nranks > MAX_RANKS || rank < 0 || rank >= nranks)
    return fail(MTFC_ERR_SHAPE, "gemm_allreduce: %d ranks (2..%d supported), rank %d", nranks,
                MAX_RANKS, rank);
  if (!stage || !out || !flags || !ctl) return fail(MTFC_ERR_SHAPE, "gemm_allreduce: null argument");
  if (d->batch != 1 || d->out_dtype != MTFC_BF16 || d->c_n != 1 || d->c_m != d->n || d->n % 8 != 0)
    return fail(MTFC_ERR_UNSUPPORTED,
                "gemm_allreduce: needs batch 1 and a dense row-major bf16 [m, n] output with n a "
                "multiple of 8");
  if (d->epilogue != MTFC_EPILOGUE_NONE)
    return fail(MTFC_ERR_UNSUPPORTED, "gemm_allreduce: no epilogue on a partial sum");
  for (int p = 0; p < nranks; ++p)
    if (!stage[p] || !out[p] || !flags[p] || !aligned16(stage[p]) || !aligned16(out[p]))
      return fail(MTFC_ERR_SHAPE, "gemm_allreduce: buffer of rank %d missing or not 16-byte aligned", p);
  if (!gemm_tcgen05_eligible(d, a, b, stage[rank]))
    return fail(MTFC_ERR_UNSUPPORTED, "gemm_allreduce: operands not eligible for the tcgen05 path");
  const int pair_clusters = max_fused_clusters();
  if (pair_clusters < 1) return fail(MTFC_ERR_CUDA, "gemm_allreduce: no room for 2-CTA clusters");
  const int a_major = classify(d->m, d->k, d->a_m, d->a_k, 1, 0);
  const int b_major = classify(d->n, d->k, d->b_n, d->b_k, 1, 0);
  if (a_major < 0 || b_major < 0) return fail(MTFC_ERR_SHAPE, "operand layout not TMA-able");
  CUtensorMap map_a, map_b;
  int rc;
  if (a_major == 0)
    rc = encode_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, d->k, d->m, 1, d->a_m, 0, BK, BM,
                    "A (K-major)");
  else
    rc = encode_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a, d->m, d->k, 1, d->a_k, 0, 64, BK,
                    "A (M-major)");
  if (rc != MTFC_OK) return rc;
  if (b_major == 0)
    rc = encode_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b, d->k, d->n, 1, d->b_n, 0, BK,
                    BN / 2, "B (K-major)");
  else
    rc = encode_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, b, d->n, d->k, 1, d->b_k, 0, 64, BK,
                    "B (N-major)");
  if (rc != MTFC_OK) return rc;

  GemmArgs args;
  args.m = (int)d->m;
  args.n = (int)d->n;
  args.k = (int)d->k;
  args.batch = 1;
  args.tiles_m = (int)((d->m + 2 * BM - 1) / (2 * BM));
  args.tiles_n = (int)((d->n + BN - 1) / BN);
  args.a_mn_major = a_major;
  args.b_mn_major = b_major;
  args.a_batched = 0;
  args.b_batched = 0;
  args.relu = 0;
  args.out_f32 = 0;
  args.status = device_status_word();
  args.progress = nullptr;
  if (args.tiles_m > FLAG_DONE)
    return fail(MTFC_ERR_UNSUPPORTED, "gemm_allreduce: more than %d row blocks", FLAG_DONE);

  FusedArgs fa;
  memset(&fa, 0, sizeof(fa));
  fa.blocks_per_rank = (args.tiles_m + nranks - 1) / nranks;
  const long long stage_rows = (long long)nranks * fa.blocks_per_rank * 2 * BM;
  for (int p = 0; p < nranks; ++p) {
    rc = encode_map(&fa.stage_map[p], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, stage[p], d->n, stage_rows,
                    1, d->n, 0, 64, 32, "staging buffer");
    if (rc != MTFC_OK) return rc;
    fa.out[p] = static_cast<uint8_t*>(out[p]);
    fa.flags[p] = static_cast<uint32_t*>(flags[p]);
  }
  if (exchange < EXCHANGE_PUSH || exchange > EXCHANGE_MULTIMEM)
    return fail(MTFC_ERR_SHAPE, "gemm_allreduce: unknown exchange form %d", exchange);
  if (exchange == EXCHANGE_MULTIMEM && (!mc_stage || !mc_out))
    return fail(MTFC_ERR_SHAPE, "gemm_allreduce: the multimem exchange needs both multicast addresses");
  fa.exchange = exchange;
  if (exchange == EXCHANGE_MULTIMEM) {
    if (!aligned16(mc_stage) || !aligned16(mc_out))
      return fail(MTFC_ERR_SHAPE, "gemm_allreduce: multicast addresses must be 16-byte aligned");
    fa.mc_stage = static_cast<const uint8_t*>(mc_stage);
    fa.mc_out = static_cast<uint8_t*>(mc_out);
  }
  if (exchange != EXCHANGE_PUSH) {
    rc = encode_map(&fa.part_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, stage[rank], d->n,
                    (long long)args.tiles_m * 2 * BM, 1, d->n, 0, 64, 32, "partial-product buffer");
    if (rc != MTFC_OK) return rc;
  }
  for (int p = 0; p < nranks; ++p) fa.stage_all[p] = static_cast<const uint8_t*>(stage[p]);
  fa.stage = static_cast<const uint8_t*>(stage[rank]);
  fa.ctl = static_cast<uint32_t*>(ctl);
  fa.rank = rank;
  fa.nranks = nranks;
  fa.wait_cycles = g_peer_wait_cycles;
  const long long num_tiles = (long long)args.tiles_m * args.tiles_n;
  // every cluster must be resident at once: the comm warps wait on other CTAs' products
  const long long clusters = num_tiles < pair_clusters ? num_tiles : pair_clusters;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
  cfg.blockDim = dim3(NUM_THREADS_FUSED, 1, 1);
  cfg.dynamicSmemBytes = SMEM2F_ALLOC;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // A cooperative launch starts only when the whole grid can be resident at once,
  // which is what the comm warps' waits on other CTAs' products rely on; without it
  // a kernel of another stream could keep some clusters off the GPU.  Where the
  // driver refuses the attribute together with clusters, the plain launch (grid
  // sized from the occupancy query above) is used from then on.
  attr[1].id = cudaLaunchAttributeCooperative;
  attr[1].val.cooperative = 1;
  cfg.attrs = attr;
  g_cooperative_launched = 1;
  if (g_cooperative_ok) {
    cfg.numAttrs = 2;
    cudaError_t e = cudaLaunchKernelEx(&cfg, einsum_gemm_allreduce_2cta, map_a, map_b, args, fa);
    if (e == cudaSuccess) return MTFC_OK;
    (void)cudaGetLastError();
    g_cooperative_ok = 0;
  }
  cfg.numAttrs = 1;
  MTFC_CUDA(cudaLaunchKernelEx(&cfg, einsum_gemm_allreduce_2cta, map_a, map_b, args, fa));
  return MTFC_OK;
}

// 1: the fused kernel is launched cooperatively; 0: the driver refused that and
// plain launches are used; -1: no launch has been made yet.
int gemm_allreduce_cooperative() { return g_cooperative_launched ? g_cooperative_ok : -1; }

}  // namespace mtfc
