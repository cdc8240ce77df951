/*
 * libmtfc — C ABI of the sm_100a kernels behind CudaMeshImpl.
 *
 * Mesh TensorFlow itself has no native boundary: a MeshImpl is a Python class
 * (mesh_tensorflow/ops.py:867-1340) whose slice arithmetic is delegated to
 * TensorFlow ops.  This header is the boundary that takes TensorFlow's place:
 * each entry point names the reference call site whose per-slice arithmetic it
 * replaces.  The only intended caller is the Python class CudaMeshImpl through
 * ctypes; a reference-side binding would be the same ctypes stub.
 *
 * Conventions
 *   - every function returns MTFC_OK (0) or a negative MTFC_ERR_* code and
 *     never throws, aborts or traps; mtfc_last_error() gives the message of the
 *     calling thread's last failure;
 *   - all buffers are caller-owned device pointers valid on the current CUDA
 *     device; nothing is retained past the stream work a call enqueues;
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream);
 *     calls are asynchronous unless stated otherwise;
 *   - strides are in elements, sizes in elements;
 *   - kernels that wait on barriers give up after a bounded time and record a
 *     code in a per-device status word that mtfc_device_status() returns.
 */
#ifndef MTFC_H_
#define MTFC_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MTFC_OK 0
#define MTFC_ERR_CUDA (-1)        /* a CUDA runtime/driver call failed          */
#define MTFC_ERR_SHAPE (-2)       /* sizes/strides/alignment not acceptable     */
#define MTFC_ERR_TIMEOUT (-3)     /* a device-side bounded wait ran out         */
#define MTFC_ERR_UNSUPPORTED (-4) /* dtype/op combination not implemented       */

#define MTFC_F32 0
#define MTFC_BF16 1
#define MTFC_I32 2

#define MTFC_MAX_DIMS 8

/* ---- library state ------------------------------------------------------ */

/* Message of the calling thread's most recent failure ("" if none). */
const char* mtfc_last_error(void);

/* ABI version of this build. */
int mtfc_version(void);

/* Number of kernels this library has launched in this process so far. */
int64_t mtfc_launch_count(void);

/* Synchronises the current device, then returns and clears its status word:
 * MTFC_OK, or MTFC_ERR_TIMEOUT if a kernel's bounded wait gave up. */
int mtfc_device_status(void);

/* ---- K1: slice contraction (GEMM) --------------------------------------- */
/*
 * Replaces tf.einsum on one processor's slices as called from
 * MeshImpl.einsum (ops.py:1331-1340) via _einsum_helper (ops.py:2816-2822).
 * The host maps a two-operand einsum onto
 *     C[b, m, n] = epilogue( sum_k A[b, m, k] * B[b, k, n] )
 * and passes the element strides each merged dimension has in the operands'
 * own named-dim order, so no transposed copy is made.
 *
 * With bf16 operands whose layout a TMA tensor map can describe (one of the
 * two strides of each operand is 1, the other and the batch stride are
 * multiples of 8 elements, C rows are contiguous) the contraction runs on the
 * tcgen05 tensor cores with fp32 accumulation in TMEM; everything else (fp32,
 * int32, awkward strides) runs on the FFMA kernel with fp32 accumulation.
 */
typedef struct {
  int64_t batch, m, n, k;
  int64_t a_batch, a_m, a_k; /* element strides of A                          */
  int64_t b_batch, b_k, b_n; /* element strides of B                          */
  int64_t c_batch, c_m, c_n; /* element strides of C                          */
  int32_t in_dtype;          /* MTFC_BF16 / MTFC_F32 / MTFC_I32 (A and B)     */
  int32_t out_dtype;         /* MTFC_BF16 / MTFC_F32 / MTFC_I32               */
  int32_t epilogue;          /* 0 = none, 1 = ReLU (tf.nn.relu, ops.py:1921)  */
  int32_t force_path;        /* 0 = auto, 1 = tcgen05 or fail, 2 = FFMA       */
} mtfc_gemm_desc;

#define MTFC_EPILOGUE_NONE 0
#define MTFC_EPILOGUE_RELU 1

int mtfc_gemm(const mtfc_gemm_desc* desc, const void* a, const void* b, void* c,
              void* stream);

/* 1 if mtfc_gemm would take the tcgen05 path for this problem, 0 if FFMA,
 * negative on invalid descriptors. Launches nothing. */
int mtfc_gemm_uses_tensor_cores(const mtfc_gemm_desc* desc, const void* a,
                                const void* b, const void* c);

#ifdef __cplusplus
}
#endif
#endif /* MTFC_H_ */
