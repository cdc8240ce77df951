// Stream-side building blocks of the pipelined einsum + allreduce: the GEMM
// runs un-chunked on the compute stream and reports row-block progress; a
// communication stream moves the partial sums with the copy engines (which
// share no SM resource with the GEMM and overlap it fully) and uses the three
// small kernels below between the copies:
//
//   wait_counters   one thread per counter polls until every counter of a range
//                   has reached epoch * per_epoch (epoch = this waiter's own
//                   launch count, kept on the device so that a recorded launch
//                   can be replayed), for at most a cycle budget; on expiry it
//                   records MTFC_ERR_TIMEOUT in the device status word
//   signal_peers    one release-add on the same counter of every listed peer
//   add_n_bf16      dst = sum of up to eight bf16 sources, fp32 accumulation in
//                   source order, one rounding (for two sources: the correctly
//                   rounded sum)
//
// All three are tiny grids with no shared memory, so they fit on SMs that a
// persistent GEMM CTA already occupies.  They stand, together with the copies,
// for the allreduce of PlacementMeshImpl (placement_mesh_impl.py:200-212,
// 358-455) in the one-process-per-GPU setting.

#include "common.cuh"

namespace mtfc {
namespace {

constexpr int kMaxPeers = 8;

struct PeerFlags {
  uint32_t* ptr[kMaxPeers];
};
struct AddSources {
  const uint4* ptr[kMaxPeers];
};

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void wait_counters_kernel(const uint32_t* __restrict__ counters, int count,
                                     uint32_t per_epoch, uint32_t* __restrict__ epoch_counter,
                                     long long limit_cycles, int* __restrict__ status) {
  __shared__ uint32_t epoch;
  if (threadIdx.x == 0) {
    epoch = *epoch_counter + 1u;
    *epoch_counter = epoch;
  }
  __syncthreads();
  const uint32_t target = epoch * per_epoch;
  const long long t0 = clock64();
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    for (;;) {
      if ((int32_t)(ld_acquire_sys_u32(counters + i) - target) >= 0) break;
      if (clock64() - t0 > limit_cycles) {
        if (status) atomicExch(status, MTFC_ERR_TIMEOUT);
        break;
      }
      __nanosleep(200);
    }
  }
}

__global__ void signal_peers_kernel(PeerFlags flags, int n, long long index) {
  if ((int)threadIdx.x < n)
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(flags.ptr[threadIdx.x] + index),
                 "r"(1u)
                 : "memory");
}

__global__ void __launch_bounds__(256)
add_n_bf16_kernel(AddSources src, int n, uint4* __restrict__ dst, long long nvec) {
  const long long step = (long long)gridDim.x * blockDim.x;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += step) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < n; ++s) {
      const uint4 x = src.ptr[s][v];
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] += __uint_as_float(w[e] << 16);
        acc[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
      }
    }
    uint4 o;
    __nv_bfloat162 h;
    h = __floats2bfloat162_rn(acc[0], acc[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(acc[2], acc[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(acc[4], acc[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
    h = __floats2bfloat162_rn(acc[6], acc[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
    dst[v] = o;
  }
}

long long g_pipeline_wait_cycles = 6000000000LL;  // ~3 s

}  // namespace
}  // namespace mtfc

using namespace mtfc;

extern "C" {

int mtfc_pipeline_set_wait_ms(int ms) {
  g_pipeline_wait_cycles = ms > 0 ? (long long)ms * 2000000LL : 6000000000LL;
  return MTFC_OK;
}

int mtfc_wait_counters(const uint32_t* counters, int32_t count, uint32_t per_epoch,
                       uint32_t* epoch_counter, void* stream) {
  if (!counters || !epoch_counter || count < 1 || count > 65536)
    return fail(MTFC_ERR_SHAPE, "wait_counters: bad arguments");
  const int threads = count < 256 ? ((count + 31) / 32) * 32 : 256;
  wait_counters_kernel<<<1, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      counters, count, per_epoch, epoch_counter, g_pipeline_wait_cycles, device_status_word());
  MTFC_LAUNCH_CHECK("wait_counters_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_signal_peers(void* const* peer_counters, int32_t n, int64_t index, void* stream) {
  if (!peer_counters || n < 1 || n > kMaxPeers || index < 0)
    return fail(MTFC_ERR_SHAPE, "signal_peers: bad arguments");
  PeerFlags f;
  for (int i = 0; i < kMaxPeers; ++i)
    f.ptr[i] = i < n ? static_cast<uint32_t*>(peer_counters[i]) : nullptr;
  for (int i = 0; i < n; ++i)
    if (!f.ptr[i]) return fail(MTFC_ERR_SHAPE, "signal_peers: null counter array %d", i);
  signal_peers_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, n, index);
  MTFC_LAUNCH_CHECK("signal_peers_kernel");
  count_launch(1);
  return MTFC_OK;
}

int mtfc_add_n_bf16(const void* const* sources, int32_t n, void* dst, int64_t elements,
                    void* stream) {
  if (!sources || !dst || n < 1 || n > kMaxPeers || elements < 0)
    return fail(MTFC_ERR_SHAPE, "add_n: bad arguments");
  if (elements == 0) return MTFC_OK;
  if (elements % 8 != 0) return fail(MTFC_ERR_SHAPE, "add_n: element count must be a multiple of 8");
  AddSources s;
  for (int i = 0; i < kMaxPeers; ++i) s.ptr[i] = i < n ? static_cast<const uint4*>(sources[i]) : nullptr;
  for (int i = 0; i < n; ++i)
    if (!s.ptr[i] || (reinterpret_cast<uintptr_t>(s.ptr[i]) & 15))
      return fail(MTFC_ERR_SHAPE, "add_n: source %d missing or not 16-byte aligned", i);
  if (reinterpret_cast<uintptr_t>(dst) & 15) return fail(MTFC_ERR_SHAPE, "add_n: dst not 16-byte aligned");
  const long long nvec = elements / 8;
  // at most two small CTAs per SM: they run beside a GEMM CTA
  add_n_bf16_kernel<<<grid_for(nvec, 256 * 4, 2), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      s, n, static_cast<uint4*>(dst), nvec);
  MTFC_LAUNCH_CHECK("add_n_bf16_kernel");
  count_launch(1);
  return MTFC_OK;
}

}  // extern "C"
