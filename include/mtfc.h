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
  int32_t force_path;        /* 0 = auto, 1 = tcgen05 or fail, 2 = FFMA,
                                3 / 4 = tcgen05 single-CTA / CTA-pair kernel   */
} mtfc_gemm_desc;

#define MTFC_EPILOGUE_NONE 0
#define MTFC_EPILOGUE_RELU 1

int mtfc_gemm(const mtfc_gemm_desc* desc, const void* a, const void* b, void* c,
              void* stream);

/* 1 if mtfc_gemm would take the tcgen05 path for this problem, 0 if FFMA,
 * negative on invalid descriptors. Launches nothing. */
int mtfc_gemm_uses_tensor_cores(const mtfc_gemm_desc* desc, const void* a,
                                const void* b, const void* c);

/*
 * mtfc_gemm fused with the SUM allreduce of its output over `nranks` GPUs, one
 * process per GPU: replaces the pair "local einsum, then allreduce over the mesh
 * axes of the contracted split dims" of EinsumOperation.lower (ops.py:2867-2873;
 * allreduce itself: placement_mesh_impl.py:358-391).  One kernel launch per rank.
 * Row blocks of 256 output rows are owned round-robin; every rank's epilogue
 * stores its partial tiles into the owner's staging buffer (peer memory), and
 * four extra warps in every CTA add the nranks copies of the owned blocks (packed
 * bf16 additions as a balanced tree over the ranks for 2, 4 or 8 ranks - the
 * correctly rounded sum for 2; fp32 accumulation with one rounding otherwise) and
 * write the sums into every rank's `out` buffer while the MMA pipeline is still
 * multiplying the later blocks.  Every rank receives the same bits.  All ranks
 * of the group must call it in the same order with the same shapes.
 *
 * desc: batch 1, bf16 in, bf16 out, c_m == n, c_n == 1, n % 8 == 0, no epilogue.
 * stage_ptrs / out_ptrs / flag_ptrs: nranks device addresses each, index r =
 * rank r's buffer as mapped into THIS process (peer-accessible: CUDA VMM or IPC
 * mappings).  stage is mtfc_gemm_allreduce_stage_bytes(m, n, nranks) bytes, out
 * is m*n bf16, flags is mtfc_gemm_allreduce_flag_bytes() bytes zeroed once before
 * first use and owned by this (m, n, group) from then on.  ctl: 16 bytes of this
 * rank's own device memory, zeroed once.  Waits on peers are bounded (~3 s); a
 * peer that never arrives gives MTFC_ERR_TIMEOUT in mtfc_device_status, after
 * which the buffers must be re-created.
 */
int mtfc_gemm_allreduce_flag_bytes(void);
/* Limit, in milliseconds at a nominal 2 GHz, of each wait on another rank inside
 * later mtfc_gemm_allreduce launches of this process; ms <= 0 restores the
 * default (~3 s).  A job whose ranks can be further apart than that when they
 * reach the launch (first-use set-up on one rank, a long host pause) should raise
 * it; a test that wants to see the time-out path lowers it. */
int mtfc_gemm_allreduce_set_wait_ms(int ms);
/* How the fused kernel is launched: 1 = cooperatively (the whole grid is
 * guaranteed resident, which its waits between CTAs rely on), 0 = the driver
 * refused a cooperative cluster launch and plain launches are used, -1 = not
 * launched yet. */
int mtfc_gemm_allreduce_cooperative(void);
int64_t mtfc_gemm_allreduce_stage_bytes(int64_t m, int64_t n, int nranks);
int mtfc_gemm_allreduce(const mtfc_gemm_desc* desc, const void* a, const void* b,
                        void* const* stage_ptrs, void* const* out_ptrs,
                        void* const* flag_ptrs, void* ctl, int rank, int nranks,
                        void* stream);

/* The same with a choice of how the partial products travel:
 *   MTFC_EXCHANGE_PUSH      as mtfc_gemm_allreduce: the epilogue stores each tile into
 *                           the owner's staging buffer over NVLink.
 *   MTFC_EXCHANGE_PULL      every rank keeps its partial product in its own staging
 *                           buffer, so the GEMM's epilogue never waits on NVLink; the
 *                           owner's reduction warps read the other ranks' copies with
 *                           peer loads.  Same bytes on the links as PUSH.
 *   MTFC_EXCHANGE_MULTIMEM  partial products local as for PULL; `stage_multicast` and
 *                           `out_multicast` are the multicast (NVLS) addresses of the
 *                           group's staging and output buffers - the same allocations
 *                           as stage_ptrs / out_ptrs, each bound to one multicast
 *                           object.  The owner of a row block reads the fp32-accumulated
 *                           sum of all ranks' copies with multimem.ld_reduce (the switch
 *                           adds) and writes it to all ranks with multimem.st: (1 + 1/n)
 *                           times the output's bytes per direction per GPU, against
 *                           2(n-1)/n for the other two - less from n = 4 up.
 * The multicast addresses are ignored by the first two forms. */
#define MTFC_EXCHANGE_PUSH 0
#define MTFC_EXCHANGE_PULL 1
#define MTFC_EXCHANGE_MULTIMEM 2
int mtfc_gemm_allreduce_ex(const mtfc_gemm_desc* desc, const void* a, const void* b,
                           void* const* stage_ptrs, void* const* out_ptrs, void* const* flag_ptrs,
                           void* ctl, int rank, int nranks, int exchange,
                           const void* stage_multicast, void* out_multicast, void* stream);

/* Pipelined form of "local einsum, then allreduce" (ops.py:2867-2873,
 * placement_mesh_impl.py:200-212): the GEMM runs un-chunked and counts finished
 * row blocks; a second stream moves the partial sums with the copy engines,
 * which overlap the GEMM fully, and reduces them with small kernels.
 *   mtfc_gemm_with_progress: mtfc_gemm on the CTA-pair tensor-core kernel (bf16,
 *     batch 1, m >= 256) that also increments progress[rb] once per epilogue warp
 *     and tile of 256-row block rb when the tile's rows are in memory:
 *     8 * ceil(n / 256) increments per launch complete a row block.  The array is
 *     never reset; consumers count launches.
 *   mtfc_wait_counters: a one-CTA kernel that returns when counters[0..count) have
 *     all reached (launches of this waiter so far, kept in *epoch_counter) *
 *     per_epoch.  The wait is bounded (mtfc_pipeline_set_wait_ms, default ~3 s);
 *     when it runs out MTFC_ERR_TIMEOUT is recorded for mtfc_device_status and
 *     the kernel returns.
 *   mtfc_signal_peers: adds 1 (release, system scope) to peer_counters[i][index]
 *     for i < n <= 8 - after everything enqueued earlier on the stream.
 *   mtfc_add_n_bf16: dst = sum of n <= 8 bf16 arrays, fp32 accumulation in source
 *     order, one rounding; elements a multiple of 8, 16-byte aligned buffers. */
int mtfc_gemm_with_progress(const mtfc_gemm_desc* desc, const void* a, const void* b, void* c,
                            uint32_t* progress, void* stream);
int mtfc_pipeline_set_wait_ms(int ms);
int mtfc_wait_counters(const uint32_t* counters, int32_t count, uint32_t per_epoch,
                       uint32_t* epoch_counter, void* stream);
int mtfc_signal_peers(void* const* peer_counters, int32_t n, int64_t index, void* stream);
int mtfc_add_n_bf16(const void* const* sources, int32_t n, void* dst, int64_t elements,
                    void* stream);

/* MeshImpl.alltoall (placement_mesh_impl.py:228-242, 490-510) between the ranks
 * of one mesh-axis group as one kernel over peer-mapped memory: every rank
 * reads its slice in place and stores part r of it straight into rank r's
 * output buffer where the concatenation puts it - no pack and no unpack pass.
 * Every rank of the group makes the same call, with
 *   src              its slice (16-byte aligned),
 *   peer_out[i]      rank i's output buffer as mapped into this process,
 *   peer_flags[i]    rank i's flag array (mtfc_alltoall_peer_flag_bytes bytes,
 *                    zeroed once when allocated),
 *   dims / strides   one part described as `ndims` <= 4 leading extents with their
 *                    byte strides in the source slice and in the output, followed
 *                    by a row of row_bytes that is contiguous in both,
 *   src_part_stride  part r starts r * src_part_stride bytes into src,
 *   dst_part_stride  the part received from rank s lands s * dst_part_stride
 *                    bytes into the output,
 *   slot, slot_stride  every rank's buffer is a row of equal slots slot_stride bytes
 *                    apart; this rank's result is wanted in slot `slot` of its own
 *                    buffer (the peers learn the number through the hand-shake, so
 *                    each rank chooses a slot that is free on its side),
 *   ctl              two zero-initialised uint32 of this rank (launch count, ticket).
 * All byte counts are multiples of 16.  The kernel waits for the peers' "buffer
 * free" signal before it stores and for their "stored" signal before it ends;
 * both waits are bounded (mtfc_alltoall_peer_set_wait_ms, default ~3 s) and raise
 * MTFC_ERR_TIMEOUT for mtfc_device_status when they run out. */
int64_t mtfc_alltoall_peer_flag_bytes(void);
int mtfc_alltoall_peer_set_wait_ms(int ms);
/* CTAs per SM the copy grid is capped at (1..8, default 4): fewer leave room for a GEMM
 * that runs beside it on another stream. */
int mtfc_alltoall_peer_set_ctas_per_sm(int ctas);
int mtfc_alltoall_peer(const void* src, void* const* peer_out, void* const* peer_flags,
                       int32_t nranks, int32_t rank, int32_t ndims, const int64_t* dims,
                       const int64_t* src_strides, const int64_t* dst_strides, int64_t row_bytes,
                       int64_t src_part_stride, int64_t dst_part_stride, int32_t slot,
                       int64_t slot_stride, uint32_t* ctl, void* stream);

/* K1f on the tensor cores: fp32 [batch, rows, k] (element strides s_*) -> bf16
 * [batch, rows, 6k], every value split into three bf16 terms laid along K
 * (pattern 0 for the left operand, 1 for the right) so that one mtfc_gemm over
 * 6k with fp32 output equals the fp32 contraction to ~1e-6 relative.  Serves the
 * same tf.einsum call as mtfc_gemm (ops.py:1331-1340) for float32 tensors. */
int mtfc_split_bf16x3(const float* src, int64_t s_batch, int64_t s_row, int64_t s_k, void* dst_bf16,
                      int64_t batch, int64_t rows, int64_t k, int pattern, void* stream);

/* ---- K8: slice-local array operations ----------------------------------- */
/*
 * The op-by-op lowering applies TensorFlow ops to slices inside
 * MeshImpl.slicewise closures.  These entry points stand for them:
 *   mtfc_unary            tf.nn.relu / exp / log / negative / reciprocal / sqrt /
 *                         rsqrt / square / tanh / sigmoid / sign / logical_not and
 *                         tf.cast (ops.py:1727-1962); IDENTITY with different
 *                         dtypes is the cast, NONZERO the cast to bool
 *   mtfc_binary           tf.add / subtract / multiply / divide / maximum /
 *                         minimum / floordiv / mod / comparisons / logical ops
 *                         with broadcasting (ops.py:2044-2200); a stride of 0
 *                         broadcasts; b == NULL uses `scalar_b`
 *   mtfc_broadcast_reduce broadcast-multiply-reduce form of einsum
 *                         (ops.py:2805-2814) and tf.reduce_sum / max / min over
 *                         any axes with an output permutation (ops.py:2267-2338)
 *   mtfc_topk_last        tf.math.reduce_max + argmax, tf.math.top_k on the last
 *                         axis (ops.py:4937-4942); ties go to the lowest index;
 *                         `values` may be NULL
 *   mtfc_gather_last      tf.gather(..., batch_dims = rank-1) (ops.py:4956-4958)
 *   mtfc_one_hot          tf.one_hot (ops.py:3843-3848); out-of-range -> all off
 *   mtfc_fill             tf.zeros / constants / tf.range: out[i] = value + step*i
 * bool tensors are int32 0/1.  Outputs are contiguous.
 */
#define MTFC_UNARY_IDENTITY 0
#define MTFC_UNARY_RELU 1
#define MTFC_UNARY_EXP 2
#define MTFC_UNARY_LOG 3
#define MTFC_UNARY_NEGATIVE 4
#define MTFC_UNARY_RECIPROCAL 5
#define MTFC_UNARY_SQRT 6
#define MTFC_UNARY_RSQRT 7
#define MTFC_UNARY_SQUARE 8
#define MTFC_UNARY_TANH 9
#define MTFC_UNARY_SIGMOID 10
#define MTFC_UNARY_SIGN 11
#define MTFC_UNARY_LOGICAL_NOT 12
#define MTFC_UNARY_NONZERO 13

#define MTFC_BINARY_ADD 0
#define MTFC_BINARY_SUB 1
#define MTFC_BINARY_MULTIPLY 2
#define MTFC_BINARY_DIVIDE 3
#define MTFC_BINARY_MAXIMUM 4
#define MTFC_BINARY_MINIMUM 5
#define MTFC_BINARY_FLOORDIV 6
#define MTFC_BINARY_MOD 7
#define MTFC_BINARY_LESS 8
#define MTFC_BINARY_GREATER 9
#define MTFC_BINARY_LESS_EQUAL 10
#define MTFC_BINARY_GREATER_EQUAL 11
#define MTFC_BINARY_EQUAL 12
#define MTFC_BINARY_NOT_EQUAL 13
#define MTFC_BINARY_LOGICAL_AND 14
#define MTFC_BINARY_LOGICAL_OR 15
#define MTFC_BINARY_SELECT_POSITIVE 16 /* a where b > 0, else 0: the ReLU gradient in one pass */

#define MTFC_REDUCE_SUM 0
#define MTFC_REDUCE_MAX 1
#define MTFC_REDUCE_MIN 2

int mtfc_unary(int op, const void* x, int x_dtype, void* y, int y_dtype, int64_t n, void* stream);

int mtfc_binary(int op, const void* a, const int64_t* a_strides, const void* b,
                const int64_t* b_strides, double scalar_b, void* out, int in_dtype,
                int out_dtype, int ndim, const int64_t* shape, void* stream);

/* out[o] = reduce over r of prod_k in[k][o, r].  `out_strides[k]` / `red_strides[k]`
 * give operand k's element stride along each kept / reduced axis (0 where the
 * operand lacks the axis).  Up to 4 operands; products reduce with SUM only. */
int mtfc_broadcast_reduce(int op, int n_in, const void* const* in, int in_dtype, void* out,
                          int out_dtype, int ndim_out, const int64_t* out_shape,
                          const int64_t* const* out_strides, int ndim_red,
                          const int64_t* red_shape, const int64_t* const* red_strides,
                          void* stream);

int mtfc_topk_last(const void* x, int dtype, int64_t rows, int32_t cols, int32_t k, void* values,
                   int32_t* indices, void* stream);

int mtfc_gather_last(const void* values, int dtype, const int32_t* indices, int64_t rows,
                     int32_t cols, int32_t k, void* out, void* stream);

int mtfc_one_hot(const int32_t* indices, int64_t n, int32_t depth, float on_value,
                 float off_value, void* out, int out_dtype, void* stream);

int mtfc_fill(void* out, int dtype, int64_t n, float value, float step, void* stream);

/* ---- K6: fused attention -------------------------------------------------- */
/*
 * out = softmax(scale * q.k^T + causal bias) . v for bf16 q, k, v, fp32 softmax,
 * weights rounded to bf16 before the second product; the logits are never
 * written to memory.  Replaces the einsum / add-mask / softmax / cast / einsum
 * chain of dot_product_attention (layers.py:1640-1652, transformer/attention.py:
 * 71-88).  `causal` applies the autoregressive bias of layers.py:1839-1850
 * (keys right of the query get weight exactly 0).  Tensors are logical
 * [batch, heads, length, d]; *_strides give the element strides of those four
 * axes in that order, so [b,h,l,d] and [b,l,h,d] storage are both read in place.
 * d must be 64 or 128 with stride 1; other strides multiples of 8.
 * mtfc_attention_supported returns 1 when a problem meets these conditions. */
int mtfc_attention_supported(int64_t d, const int64_t* q_strides, const int64_t* k_strides,
                             const int64_t* v_strides, const int64_t* o_strides);

/* Kernel variant mtfc_attention_fwd uses: 0 = by query length (default), 1 = one
 * 128-row query tile per CTA, 2 = two tiles per CTA with the weights kept in TMEM.
 * Process-wide; meant for tests and tuning. */
int mtfc_attention_set_variant(int variant);

int mtfc_attention_fwd(const void* q, const void* k, const void* v, void* out, int64_t batch,
                       int64_t heads, int64_t lq, int64_t lk, int64_t d, const int64_t* q_strides,
                       const int64_t* k_strides, const int64_t* v_strides,
                       const int64_t* o_strides, int32_t causal, float scale, void* stream);

/* ---- K7: strided copy ---------------------------------------------------- */
/*
 * dst[sum_d i_d * dst_strides[d]] = src[sum_d i_d * src_strides[d]] over `shape`.
 * Replaces tf.transpose / tf.slice / tf.concat / tf.split on slices: transposes in
 * _expand_dims and _reduce_helper (ops.py:5322-5343, 2267-2299), make_slices /
 * combine_slices (ops.py:1249-1305), allsplit (ops.py:1082-1109) and the split /
 * concat around allconcat and alltoall (placement_mesh_impl.py:436-440, 487,
 * 509-510).  elem_bytes is 2 or 4; rows that are contiguous on both sides move
 * as 16-byte vectors.
 */
int mtfc_copy_strided(const void* src, const int64_t* src_strides, void* dst,
                      const int64_t* dst_strides, int ndim, const int64_t* shape, int elem_bytes,
                      void* stream);

/* ---- K2-K5: top-2 mixture-of-experts routing ----------------------------- */
/*
 * Replace the op chain of _top_2_gating (transformer/moe.py:1380-1513) and the
 * dense one-hot dispatch / combine einsums (moe.py:443-447, 509-510).
 * Tokens are [groups, group_size]; groups are independent; within a group
 * tokens are served in index order; ties go to the lowest expert index.
 */
#define MTFC_MOE_POLICY_ALL 0       /* moe_second_policy "all"       */
#define MTFC_MOE_POLICY_NONE 1      /* "none"                        */
#define MTFC_MOE_POLICY_THRESHOLD 2 /* "threshold": gate_2 > thr     */
#define MTFC_MOE_POLICY_RANDOM 3    /* "random": noise < gate_2/thr  */
#define MTFC_MOE_POLICY_SWITCH 4    /* top-1 routing (_switch_gating, moe.py:1184-1309):
                                       no second expert, gate_1 is the raw softmax
                                       output (not renormalised), gate_2 = 0 */

/* fp32 gate kernel [m, experts] -> bf16 [m, 3*experts] = [hi | mid | lo] with
 * hi + mid + lo == w to fp32 accuracy, so x(bf16) . w runs on the tensor cores
 * (mtfc_gemm with n = 3*experts) and mtfc_moe_top2_gating sums the 3 parts.
 * Stands for the fp32 gate dense layer at moe.py:1384-1390. */
int mtfc_moe_split_gate_weights(const float* w, int64_t m, int32_t experts, void* out_bf16,
                                void* stream);

/* logits: [groups*group_size, parts*experts] fp32; the `parts` column blocks are
 * summed.  Outputs per token: expert indices, positions in the expert's buffer
 * (position >= capacity means the token did not fit), gates after
 * renormalisation and zeroed where dropped; optional raw softmax outputs;
 * per-group load-balancing loss (moe.py:1420-1424, before the mean over groups
 * and before moe_loss_coef). */
int mtfc_moe_top2_gating(const float* logits, int32_t parts, int64_t groups, int32_t group_size,
                         int32_t experts, int32_t capacity, int32_t policy, float threshold,
                         const float* noise, int32_t* idx1, int32_t* idx2, int32_t* pos1,
                         int32_t* pos2, float* gate1, float* gate2, float* raw_gates,
                         float* loss_per_group, void* stream);

/* The same routing as mtfc_moe_split_gate_weights + mtfc_gemm +
 * mtfc_moe_top2_gating for bf16 activations, with the activations read once:
 * one tcgen05 kernel forms the gate logits of 128 tokens at a time in TMEM
 * (x . [hi | mid | lo] of the fp32 gate kernel) and finishes softmax, top-2
 * and gate renormalisation in registers, one thread per token; a per-group
 * scan kernel then assigns positions and applies the second-expert policy and
 * the capacity (moe.py:1380-1496).
 *   mtfc_moe_gate_fused_supported: 1 when d_model `m` is a multiple of 8 and
 *     2 <= experts <= 64, else 0 (use the three-call form then).
 *   mtfc_moe_gate_padded_experts: EP, experts rounded up to 16, 32 or 64.
 *   mtfc_moe_gate_prepare: fp32 gate kernel [m, experts] -> bf16 [3*EP, m].
 *   mtfc_moe_gate_scratch_bytes: size of the caller-owned `scratch` (per-tile
 *     column sums of the raw gates, from which the loss is formed).
 *   mtfc_moe_gate_top2: x [groups*group_size, m] bf16; outputs as
 *     mtfc_moe_top2_gating; `loss_mean` (optional) receives the sum of
 *     loss_per_group divided by num_groups_total (the groups of all slices, so
 *     that per-slice values add up to the mean over all groups); `slot_table`
 *     (optional) receives what mtfc_moe_slot_table would compute from the outputs. */
int mtfc_moe_gate_fused_supported(int64_t m, int32_t experts);
int32_t mtfc_moe_gate_padded_experts(int32_t experts);
int64_t mtfc_moe_gate_scratch_bytes(int64_t groups, int32_t group_size, int32_t experts);
int mtfc_moe_gate_prepare(const float* w, int64_t m, int32_t experts, void* w3t_bf16, void* stream);
int mtfc_moe_gate_top2(const void* x_bf16, const void* w3t_bf16, int64_t groups, int32_t group_size,
                       int64_t m, int32_t experts, int32_t capacity, int32_t policy,
                       float threshold, const float* noise, int32_t* idx1, int32_t* idx2,
                       int32_t* pos1, int32_t* pos2, float* gate1, float* gate2, float* raw_gates,
                       float* loss_per_group, float* loss_mean, int64_t num_groups_total,
                       int32_t* slot_table, int32_t round_gates_to_bf16, void* scratch,
                       int64_t scratch_bytes, void* stream);

/* table[g, e, c] = token routed to slot c of expert e in group g, or -1.
 * With round_gates_to_bf16 a token whose gate rounds to 0 in bfloat16 is not
 * dispatched (the reference derives dispatch from the rounded combine tensor,
 * moe.py:1507-1511). */
int mtfc_moe_slot_table(const int32_t* idx1, const int32_t* idx2, const int32_t* pos1,
                        const int32_t* pos2, const float* gate1, const float* gate2,
                        int64_t groups, int32_t group_size, int32_t experts, int32_t capacity,
                        int32_t round_gates_to_bf16, int32_t* table, void* stream);

/* x: [outer, groups_per_outer, group_size, row] -> out: [outer, experts,
 * groups_per_outer, capacity, row]; rows of `row_bytes` bytes (multiple of 16);
 * empty slots are zero rows. */
int mtfc_moe_dispatch(const void* x, const int32_t* table, void* out, int64_t outer,
                      int64_t groups_per_outer, int32_t group_size, int32_t experts,
                      int32_t capacity, int64_t row_bytes, void* stream);

/* Same result as mtfc_moe_slot_table followed by mtfc_moe_dispatch, for callers
 * that may not allocate device memory.  This entry point has no counterpart in
 * the reference.  It is meant for hosts whose device memory is planned once at
 * start-up and then frozen — a serving process that has handed every remaining
 * byte to its own pools, or code on a latency-critical path where a cudaMalloc
 * (which can fail, and which stalls the whole device while it runs) is not
 * acceptable.  The (group, expert, slot) -> token table that the two-call form
 * takes from the caller lives here in a fixed array inside the library image:
 * 1,048,576 entries (4 MiB), held by every GPU that loads the library until the
 * process exits.  The caller still owns x, the routing arrays and out.
 *   - groups*experts*capacity above 1,048,576 is rejected with MTFC_ERR_SHAPE;
 *     nothing is launched.  Use the two-call form with your own table then.
 *   - The first call on each device looks up the array's device address, with
 *     that device current; make that first call before starting any stream
 *     capture on the device.
 *   - No cudaMalloc, cudaFree or allocating library routine is called.
 *   - All calls on a device share the one array.  Every call rewrites the part it
 *     uses before reading it, so earlier contents never leak into a result, but
 *     two calls whose kernels overlap on the GPU (different streams) race on it:
 *     keep calls on one stream, or order them with events. */
int mtfc_moe_dispatch_noalloc(const void* x, const int32_t* idx1, const int32_t* idx2,
                              const int32_t* pos1, const int32_t* pos2, const float* gate1,
                              const float* gate2, void* out, int64_t outer,
                              int64_t groups_per_outer, int32_t group_size, int32_t experts,
                              int32_t capacity, int64_t row_bytes, int32_t round_gates_to_bf16,
                              void* stream);

/* y: [outer, experts, groups_per_outer, capacity, row] -> out: [outer,
 * groups_per_outer, group_size, row] = w1*y[i1, p1] + w2*y[i2, p2] with the gates
 * rounded to y's dtype first; fp32 arithmetic, one rounding at the store. */
int mtfc_moe_combine(const void* y, int dtype, const int32_t* idx1, const int32_t* idx2,
                     const int32_t* pos1, const int32_t* pos2, const float* gate1,
                     const float* gate2, void* out, int64_t outer, int64_t groups_per_outer,
                     int32_t group_size, int32_t experts, int32_t capacity, int64_t row_elems,
                     void* stream);

/* Backward pass of mtfc_moe_combine (the transposes of the combine einsum,
 * moe.py:509-510, that mtf's einsum gradient would form densely, ops.py:2846-2854).
 *   mtfc_moe_dispatch_weighted: d(expert outputs)[o, e, g, c, :] = w * x[o, g, s, :]
 *     for the token s in slot (e, c) of `table`, w its gate for that choice rounded
 *     to `dtype`; zero rows for empty slots.  x plays dout's role.
 *   mtfc_moe_combine_gate_grad: dgate_k[o, g, s] = <dout[o, g, s, :], y[o, i_k, g, p_k, :]>
 *     for kept choices, else 0; fp32 sums. */
int mtfc_moe_dispatch_weighted(const void* x, int dtype, const int32_t* table, const int32_t* idx1,
                               const int32_t* pos1, const float* gate1, const float* gate2,
                               void* out, int64_t outer, int64_t groups_per_outer,
                               int32_t group_size, int32_t experts, int32_t capacity,
                               int64_t row_elems, void* stream);
int mtfc_moe_combine_gate_grad(const void* y, const void* dout, int dtype, const int32_t* idx1,
                               const int32_t* idx2, const int32_t* pos1, const int32_t* pos2,
                               const float* gate1, const float* gate2, float* dgate1,
                               float* dgate2, int64_t outer, int64_t groups_per_outer,
                               int32_t group_size, int32_t experts, int32_t capacity,
                               int64_t row_elems, void* stream);

/* Backward pass of the top-2 / top-1 gating (transformer/moe.py:1384-1424, 1485-1494,
 * differentiated by the reference through its op chain): from the gate logits
 * [groups, group_size, experts] (fp32, experts <= 64), the routing decisions and the
 * gradients of gate_1, gate_2 (per token; null = none) and of the loss (a device
 * scalar; null = none) to d logits.  Indices and capacity / policy masks are
 * constants (gate_k as the forward pass returned it: 0 = dropped); the loss is
 * mean over all num_groups_total groups and experts of mean_s raw * density_1, times
 * experts^2; top1_only keeps the raw top-1 gate (no renormalisation, no gate_2). */
int mtfc_moe_gate_grad(const float* logits, const int32_t* idx1, const int32_t* idx2,
                       const float* gate1, const float* gate2, const float* dgate1,
                       const float* dgate2, const float* dloss, int64_t groups, int32_t group_size,
                       int32_t experts, int64_t num_groups_total, int32_t top1_only, float* dlogits,
                       void* stream);

/* ---- K8: row kernels of the rest of a transformer block ------------------- */
/* y[r, :] = (x[r, :] - mean) * rsqrt(var + epsilon) * scale + bias over rows of
 * `cols` contiguous elements (centered: layer_norm, layers.py:950-979), or
 * x * rsqrt(mean(x^2) + epsilon) * scale (centered = 0: RMS norm,
 * transformer/transformer.py:493-516).  scale / bias: [cols] or null.  fp32
 * statistics, one rounding at the store. */
int mtfc_norm_rows(const void* x, const void* scale, const void* bias, void* y, int dtype,
                   int64_t rows, int64_t cols, float epsilon, int32_t centered, void* stream);

/* Counter-based random fill standing for tf.random.uniform / tf.random.normal
 * inside MeshImpl.random (placement_mesh_impl.py:307-325): element i is word i % 4
 * of Philox4x32-10 block i / 4 under key `seed`, so a slice's values depend only
 * on the seed (which the mesh implementation derives from the slice's offset:
 * replicas get equal values).  normal = 0: uniform in [a, b) from the word's top
 * 24 bits; normal = 1: mean a, standard deviation b by Box-Muller. */
int mtfc_random(void* out, int dtype, int64_t n, int32_t normal, uint64_t seed, float a, float b,
                void* stream);

/* out[r, :] = table[indices[r] - first_row, :] if 0 <= indices[r] - first_row <
 * table_rows, else zeros: the row gather behind mtf.gather / layers.embedding
 * (ops.py:5231-5251, a one-hot einsum in the reference).  first_row is the
 * offset of this slice of the table when the gathered dim is split over the
 * mesh; the slices' results then add up to the full gather. */
int mtfc_gather_rows(const void* table, const int32_t* indices, void* out, int64_t rows,
                     int64_t table_rows, int32_t first_row, int64_t row_bytes, void* stream);

/* Softmax cross-entropy with hard targets over rows of `cols` logits that are the
 * columns [first_col, first_col + cols) of the vocabulary (layers.py:1062-1117,
 * reduce_logsumexp ops.py:5493-5520).  mtfc_xent_stats: per row the slice's max,
 * sum of exp(x - max) and the target's logit (0 when the target lies in another
 * slice).  Over slices: M = max of maxes, Z = sum of sums * exp(max - M),
 * log_z = log Z + M, loss = log_z - sum of picked + z_loss * log_z^2.
 * mtfc_xent_grad: dlogits = dloss * ((1 + 2 z_loss log_z) softmax - onehot(target)). */
int mtfc_xent_stats(const void* logits, int dtype, const int32_t* targets, int64_t rows, int64_t cols,
                    int32_t first_col, float* row_max, float* row_sum, float* picked, void* stream);
int mtfc_xent_grad(const void* logits, int dtype, const int32_t* targets, const float* log_z,
                   const float* dloss, float z_loss, int64_t rows, int64_t cols, int32_t first_col,
                   void* dlogits, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MTFC_H_ */
