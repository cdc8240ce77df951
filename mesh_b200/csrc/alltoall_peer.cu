// MeshImpl.alltoall between the ranks of one mesh-axis group as ONE kernel over
// peer-mapped memory (NVLink / NVSwitch), for one process per GPU.
//
// The reference's alltoall (placement_mesh_impl.py:228-242 and
// alltoall_pointtwise 490-510) cuts every slice into n parts along split_axis
// and gives part r to processor r, which concatenates what it receives along
// concat_axis in processor order.  A library alltoall needs the parts packed
// contiguously per peer before the call and unpacked into the concat layout
// after it: two more passes over the data.  Here every rank reads its slice in
// its natural layout and stores part r straight into rank r's output buffer at
// the place the concatenation gives it, so the data is read once and written
// once, remotely.
//
// Hand-shake, all on monotonically increasing uint32 counters in peer-visible
// memory (epoch = this buffer's launch number, kept on the device so that a
// recorded launch can be replayed):
//   ready  Every rank r, as its kernel starts, adds 1 to slot ready[r] at every
//          peer: "my output buffer is free: whatever read its previous contents
//          was enqueued before this launch".  A rank stores into any buffer
//          only after all of its own ready slots have reached the epoch.
//          With the signal travels the number of the slot of its buffer the rank
//          wants this call's result in (a rank's buffer is a row of equal slots;
//          the receiver alone decides which one is free), written to slot[r] at
//          every peer just before the release-add.
//   done   When a rank's last CTA has finished storing (system-scope fence,
//          ticket), it adds 1 to `done` at every peer; a rank's output is
//          complete when its `done` has reached epoch * n, which its last CTA
//          waits for before the kernel ends.
// Every wait is bounded by a cycle budget; on expiry the kernel raises
// MTFC_ERR_TIMEOUT in the device status word, skips its stores and returns.
//
// The waits are on other ranks' launches, never on other CTAs of this launch, so
// the grid needs no co-residency guarantee.

#include "common.cuh"

namespace mtfc {
namespace {

constexpr int kA2AMaxRanks = 8;
constexpr int kA2AMaxDims = 4;
constexpr int kA2AThreads = 256;
constexpr int kA2AUnroll = 4;
constexpr long long kA2AChunkBytes = (long long)kA2AThreads * 16 * kA2AUnroll * 2;  // 32 KiB per work item
constexpr int kFlagStride = 32;   // uint32 words between flags: one 128-byte line each
constexpr int kFlagDone = kA2AMaxRanks;
constexpr int kFlagSlot = kA2AMaxRanks + 1;   // slot[0..7] follow
constexpr int kFlagLines = 2 * kA2AMaxRanks + 1;

struct A2AArgs {
  const uint8_t* src;
  uint8_t* out[kA2AMaxRanks];      // every rank's output buffer (slot 0)
  uint32_t* flags[kA2AMaxRanks];   // every rank's flag array: ready[0..7], done, slot[0..7]
  uint32_t my_slot;                // where this rank wants its result
  long long slot_stride;           // bytes between the slots of a buffer
  int n, me, ndims;
  long long dims[kA2AMaxDims];     // extents of one part in front of the row
  long long sstride[kA2AMaxDims];  // their strides in the source slice, bytes
  long long dstride[kA2AMaxDims];  // their strides in the output, bytes
  long long rows;                  // product of dims
  long long row_bytes;             // contiguous in source and output, a multiple of 16
  long long src_part_stride;       // part r starts r * this into the source
  long long dst_part_stride;       // the part from rank s lands s * this into the output
  uint32_t* ctl;                   // local: [0] launches completed, [1] ticket
  long long wait_cycles;
  int* status;
};

__device__ __forceinline__ uint32_t a2a_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void a2a_red_release_sys(uint32_t* p) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(1u) : "memory");
}
__device__ __forceinline__ bool a2a_wait_ge(const uint32_t* p, uint32_t target, long long limit) {
  const long long t0 = clock64();
  for (;;) {
    if ((int32_t)(a2a_ld_acquire_sys(p) - target) >= 0) return true;
    if (clock64() - t0 > limit) return false;
    __nanosleep(100);
  }
}
__device__ __forceinline__ uint4 a2a_ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__global__ void __launch_bounds__(kA2AThreads)
alltoall_peer_kernel(const A2AArgs a) {
  __shared__ uint32_t s_epoch;
  __shared__ uint32_t s_slot[kA2AMaxRanks];
  __shared__ int s_ok, s_last;
  const int tid = threadIdx.x;
  if (tid == 0) {
    s_epoch = *reinterpret_cast<volatile uint32_t*>(a.ctl) + 1u;
    s_ok = 1;
    s_last = 0;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  // this rank's buffer is free from here on: tell everybody (itself included)
  if (blockIdx.x == 0 && tid < a.n) {
    *reinterpret_cast<volatile uint32_t*>(a.flags[tid] + (kFlagSlot + a.me) * kFlagStride) = a.my_slot;
    a2a_red_release_sys(a.flags[tid] + a.me * kFlagStride);
  }
  // ... and nobody's buffer is written before its owner said the same, and where
  if (tid < a.n) {
    if (a2a_wait_ge(a.flags[a.me] + tid * kFlagStride, epoch, a.wait_cycles))
      s_slot[tid] = *reinterpret_cast<volatile uint32_t*>(a.flags[a.me] + (kFlagSlot + tid) * kFlagStride);
    else
      s_ok = 0;
  }
  __syncthreads();
  const bool ok = s_ok != 0;

  if (ok) {
    const long long chunks = (a.row_bytes + kA2AChunkBytes - 1) / kA2AChunkBytes;
    const long long items = (long long)a.n * a.rows * chunks;
    for (long long w = blockIdx.x; w < items; w += gridDim.x) {
      // neighbouring items go to different peers; every rank starts with its successor
      const int dest = (int)((a.me + 1 + w % a.n) % a.n);
      long long rest = w / a.n;
      const long long chunk = rest % chunks;
      long long row = rest / chunks;
      long long soff = (long long)dest * a.src_part_stride;
      long long doff = (long long)a.me * a.dst_part_stride;
      for (int k = a.ndims - 1; k >= 0; --k) {
        const long long i = row % a.dims[k];
        row /= a.dims[k];
        soff += i * a.sstride[k];
        doff += i * a.dstride[k];
      }
      const long long base = chunk * kA2AChunkBytes;
      const long long len = min(kA2AChunkBytes, a.row_bytes - base);
      const uint4* s = reinterpret_cast<const uint4*>(a.src + soff + base);
      uint4* d = reinterpret_cast<uint4*>(a.out[dest] + (long long)s_slot[dest] * a.slot_stride + doff + base);
      const int nvec = (int)(len >> 4);
      for (int v0 = tid; v0 < nvec; v0 += kA2AThreads * kA2AUnroll) {
        uint4 r[kA2AUnroll];
#pragma unroll
        for (int u = 0; u < kA2AUnroll; ++u) {
          const int v = v0 + u * kA2AThreads;
          if (v < nvec) r[u] = a2a_ld_stream(s + v);
        }
#pragma unroll
        for (int u = 0; u < kA2AUnroll; ++u) {
          const int v = v0 + u * kA2AThreads;
          if (v < nvec) d[v] = r[u];
        }
      }
    }
  }

  __syncthreads();
  if (tid == 0) {
    __threadfence_system();   // this CTA's stores (ordered before by the barrier) are visible everywhere
    const unsigned t = atomicAdd(a.ctl + 1, 1u);
    __threadfence();
    s_last = (t == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (!s_last) return;
  // last CTA: every store of this rank has been made visible
  bool complete = ok;
  if (ok && tid < a.n) a2a_red_release_sys(a.flags[tid] + kFlagDone * kFlagStride);
  if (tid == 0) {
    if (ok)
      complete = a2a_wait_ge(a.flags[a.me] + kFlagDone * kFlagStride, epoch * (uint32_t)a.n, a.wait_cycles);
    if (!complete && a.status) atomicExch(a.status, MTFC_ERR_TIMEOUT);
    a.ctl[1] = 0u;
    __threadfence();
    a.ctl[0] = epoch;
  }
}

long long g_a2a_wait_cycles = 6000000000LL;  // ~3 s
int g_a2a_ctas_per_sm = 4;

}  // namespace
}  // namespace mtfc

using namespace mtfc;

extern "C" {

int64_t mtfc_alltoall_peer_flag_bytes(void) {
  return (int64_t)kFlagLines * kFlagStride * sizeof(uint32_t);
}

int mtfc_alltoall_peer_set_ctas_per_sm(int ctas) {
  g_a2a_ctas_per_sm = ctas >= 1 && ctas <= 8 ? ctas : 4;
  return MTFC_OK;
}

int mtfc_alltoall_peer_set_wait_ms(int ms) {
  g_a2a_wait_cycles = ms > 0 ? (long long)ms * 2000000LL : 6000000000LL;
  return MTFC_OK;
}

int mtfc_alltoall_peer(const void* src, void* const* peer_out, void* const* peer_flags,
                       int32_t nranks, int32_t rank, int32_t ndims, const int64_t* dims,
                       const int64_t* src_strides, const int64_t* dst_strides, int64_t row_bytes,
                       int64_t src_part_stride, int64_t dst_part_stride, int32_t slot,
                       int64_t slot_stride, uint32_t* ctl, void* stream) {
  if (!src || !peer_out || !peer_flags || !ctl)
    return fail(MTFC_ERR_SHAPE, "alltoall_peer: null argument");
  if (nranks < 1 || nranks > kA2AMaxRanks || rank < 0 || rank >= nranks)
    return fail(MTFC_ERR_SHAPE, "alltoall_peer: rank %d of %d (at most %d ranks)", rank, nranks, kA2AMaxRanks);
  if (ndims < 0 || ndims > kA2AMaxDims || (ndims > 0 && (!dims || !src_strides || !dst_strides)))
    return fail(MTFC_ERR_SHAPE, "alltoall_peer: 0..%d leading dims", kA2AMaxDims);
  if (row_bytes < 0 || row_bytes % 16 != 0 || src_part_stride % 16 != 0 || dst_part_stride % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "alltoall_peer: rows and part strides must be multiples of 16 bytes");
  if (reinterpret_cast<uintptr_t>(src) % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "alltoall_peer: source not 16-byte aligned");
  if (slot < 0 || slot_stride < 0 || slot_stride % 16 != 0)
    return fail(MTFC_ERR_SHAPE, "alltoall_peer: slot %d with stride %lld", slot, (long long)slot_stride);
  A2AArgs a;
  a.src = static_cast<const uint8_t*>(src);
  for (int i = 0; i < kA2AMaxRanks; ++i) {
    a.out[i] = i < nranks ? static_cast<uint8_t*>(peer_out[i]) : nullptr;
    a.flags[i] = i < nranks ? static_cast<uint32_t*>(peer_flags[i]) : nullptr;
    if (i < nranks && (!a.out[i] || !a.flags[i] || reinterpret_cast<uintptr_t>(a.out[i]) % 16 != 0))
      return fail(MTFC_ERR_SHAPE, "alltoall_peer: buffer of rank %d missing or not 16-byte aligned", i);
  }
  a.n = nranks; a.me = rank; a.ndims = ndims;
  a.rows = 1;
  for (int k = 0; k < kA2AMaxDims; ++k) {
    a.dims[k] = k < ndims ? dims[k] : 1;
    a.sstride[k] = k < ndims ? src_strides[k] : 0;
    a.dstride[k] = k < ndims ? dst_strides[k] : 0;
    if (k < ndims) {
      if (dims[k] < 1 || src_strides[k] % 16 != 0 || dst_strides[k] % 16 != 0)
        return fail(MTFC_ERR_SHAPE, "alltoall_peer: dim %d: extent %lld, strides %lld / %lld", k,
                    (long long)dims[k], (long long)src_strides[k], (long long)dst_strides[k]);
      a.rows *= dims[k];
    }
  }
  a.row_bytes = row_bytes;
  a.src_part_stride = src_part_stride;
  a.dst_part_stride = dst_part_stride;
  a.my_slot = (uint32_t)slot;
  a.slot_stride = slot_stride;
  a.ctl = ctl;
  a.wait_cycles = g_a2a_wait_cycles;
  a.status = device_status_word();
  const long long chunks = row_bytes > 0 ? (row_bytes + kA2AChunkBytes - 1) / kA2AChunkBytes : 0;
  const long long items = (long long)nranks * a.rows * chunks;
  // the hand-shake runs even for an empty slice: every rank of the group makes the call
  long long grid = items < 1 ? 1 : items;
  const long long cap = (long long)sm_count() * g_a2a_ctas_per_sm;
  if (grid > cap) grid = cap;
  alltoall_peer_kernel<<<(unsigned)grid, kA2AThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  MTFC_LAUNCH_CHECK("alltoall_peer_kernel");
  count_launch(1);
  return MTFC_OK;
}

}  // extern "C"
