/* C ABI of libspyre_b200.so: hand-written sm_100a kernels for torch-spyre's
 * data-parallel hot path (stick relayout in host<->device copy_, fp16
 * pointwise / reduction / softmax / layernorm / matmul).
 *
 * Conventions for every entry point
 *   - returns TS_OK (0) or a negative TS_ERR_* code; never throws, never
 *     aborts, never synchronises the device;
 *   - unless its comment says otherwise it allocates nothing: the caller owns
 *     every buffer, including scratch;
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *     stream); work is enqueued on it and the call returns;
 *   - device pointers are plain addresses in the current CUDA device's memory;
 *   - a "stick image" is the device byte image of a tensor in the generic
 *     stick layout of SpyreTensorLayout (torch_spyre/csrc/spyre_tensor_impl.cpp:
 *     39-74): for a logical [rows..., cols] fp16 tensor it is the contiguous
 *     array [ceil(cols/64)][rows...][64]; lanes past `cols` are zero.
 *
 * Each declaration cites the reference interface it stands in for.
 */
#ifndef SPYRE_B200_H_
#define SPYRE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TS_MAX_DIMS 8

enum {
  TS_OK = 0,
  TS_ERR_INVALID = -1,     /* null pointer, bad rank, negative size ...        */
  TS_ERR_UNSUPPORTED = -2, /* well-formed request this build has no kernel for */
  TS_ERR_CUDA = -3,        /* a CUDA runtime call or launch failed             */
  TS_ERR_ALIGNMENT = -4,   /* pointer or stride not aligned as the entry needs */
  TS_ERR_TOO_LARGE = -5    /* size beyond a stated maximum                      */
};

/* Human-readable text for a status code (static storage). */
const char* ts_status_string(int status);
/* ABI version of the loaded library (bumped on incompatible change). */
int ts_abi_version(void);
/* Text of the last CUDA error this thread's failing call saw, "" if none. */
const char* ts_last_cuda_error(void);

/* ---- stick relayout (the device half of host<->device copy_) -------------
 *
 * Replaces the SenDataConvert host pass + DMA that the reference builds in
 * create_dma_graph / generate_dci / get_device_stride_info
 * (torch_spyre/csrc/spyre_mem.cpp:213-279, 281-438).
 *
 * `strided` is a device-resident raw image of the host tensor's storage
 * (element strides `host_strides`, any order, in elements); `sticks` is the
 * image described by a SpyreTensorLayout (device_size / device_strides /
 * dim_map, ndev entries, outermost first).  A host dim that appears several
 * times in dim_map is split over those device dims, outermost most
 * significant.  to_sticks writes every element of the stick image (pad lanes
 * become zero); from_sticks writes exactly the host tensor's elements.
 * elem_bytes is 1, 2, 4 or 8.  Bit-exact: elements are moved, never converted.
 */
int ts_relayout_to_sticks(const void* strided, void* sticks, int elem_bytes,
                          const int64_t* host_size, const int64_t* host_strides, int rank,
                          const int64_t* device_size, const int64_t* device_strides,
                          const int32_t* dim_map, int ndev, void* stream);
int ts_relayout_from_sticks(const void* sticks, void* strided, int elem_bytes,
                            const int64_t* host_size, const int64_t* host_strides, int rank,
                            const int64_t* device_size, const int64_t* device_strides,
                            const int32_t* dim_map, int ndev, void* stream);

/* Host-buffer forms of the two calls above, i.e. copy_host_to_device /
 * copy_device_to_host (torch_spyre/csrc/spyre_mem.cpp:408-438).  `host` points
 * at the element with all-zero index; the host tensor must have non-negative
 * strides.  `staging` is a caller-owned device buffer of at least
 * ts_host_span_bytes(...) bytes.  The raw span of host storage the tensor
 * touches is copied with cudaMemcpyAsync (pinned host memory makes it
 * asynchronous) and relaid out on the device, all on `stream`.
 */
int64_t ts_host_span_bytes(int elem_bytes, const int64_t* host_size,
                           const int64_t* host_strides, int rank);
int ts_copy_host_to_sticks(const void* host, void* staging, void* sticks, int elem_bytes,
                           const int64_t* host_size, const int64_t* host_strides, int rank,
                           const int64_t* device_size, const int64_t* device_strides,
                           const int32_t* dim_map, int ndev, void* stream);
int ts_copy_sticks_to_host(const void* sticks, void* staging, void* host, int elem_bytes,
                           const int64_t* host_size, const int64_t* host_strides, int rank,
                           const int64_t* device_size, const int64_t* device_strides,
                           const int32_t* dim_map, int ndev, void* stream);

/* Pipelined forms of the two host-buffer calls.  The host span is cut along the
 * tensor's leading dim into chunks of about 8 MiB that travel through the two
 * halves of `staging`: the PCIe copy of one chunk runs on an internal copy
 * stream while the relayout kernel of the previous one runs on `stream`, and
 * the staging buffer need only hold ts_copy_staging_bytes(...) bytes (at most
 * 16 MiB) instead of the whole span.  Synchronising `stream` afterwards
 * covers the copies too.  A tensor that cannot be cut that way (rank 1, a
 * leading dim that is the stick dim or overlaps in memory, a destination with
 * gaps between its elements) takes the single-shot path above and then
 * needs staging_bytes >= ts_host_span_bytes(...) (TS_ERR_TOO_LARGE otherwise).
 * First use on a device creates that device's copy stream and four events
 * (no device memory); later calls on the device reuse them and are serialised
 * while they enqueue.  A pageable (neither pinned nor registered) host tensor
 * of 4 MiB or more is staged by the library itself rather than by the driver:
 * helper threads that live for the one call copy between it and two pinned
 * blocks of one chunk each (allocated per device on first need, at most 32 MiB
 * each) while the neighbouring chunk is on the bus; for such a tensor the
 * device-to-host call has the data in `host` when it returns, and the
 * host-to-device call no longer reads `host` after it returns; the destination
 * of such a device-to-host copy is marked for transparent huge pages
 * (madvise), so that freshly allocated memory faults in 2 MiB at a time.  Same reference
 * interfaces as above (torch_spyre/csrc/spyre_mem.cpp:408-438).
 */
int64_t ts_copy_staging_bytes(int elem_bytes, const int64_t* host_size, const int64_t* host_strides,
                              int rank);
/* The helper-thread copy the pipelined calls use for pageable host memory, on its own: copies
 * `bytes` bytes from `src` to `dst` (host pointers, not overlapping) with `threads` threads
 * (1..64) that exist only for the call.  Needs no GPU; for tests of the host logic.  No
 * counterpart in the reference. */
int ts_host_copy_selftest(void* dst, const void* src, int64_t bytes, int threads);
int ts_copy_host_to_sticks_pipelined(const void* host, void* staging, int64_t staging_bytes, void* sticks,
                                     int elem_bytes, const int64_t* host_size,
                                     const int64_t* host_strides, int rank, const int64_t* device_size,
                                     const int64_t* device_strides, const int32_t* dim_map, int ndev,
                                     void* stream);
int ts_copy_sticks_to_host_pipelined(const void* sticks, void* staging, int64_t staging_bytes, void* host,
                                     int elem_bytes, const int64_t* host_size,
                                     const int64_t* host_strides, int rank, const int64_t* device_size,
                                     const int64_t* device_strides, const int32_t* dim_map, int ndev,
                                     void* stream);

/* Stick image -> stick image for a strided view on either side, in one pass:
 * the device-side restickify behind transposed / permuted / sliced / narrowed
 * / expanded tensors.  Stands in for the reference's data-op programs
 * (2-D and 3-D transposes in 64x64 pieces and slices,
 * torch_spyre/_inductor/codegen/data_ops.py:16-189, 193-487, 490-630) and for
 * the CPU bounce of its view ops (codegen/templates/view.jinja2:40-46).
 *
 * Each side is the generic stick image of a row-major base tensor
 * (`*_base`, `*_base_rank` dims) together with a view of that base: `size`
 * (shared by both sides, `rank` dims), element strides and an element offset
 * in the base's row-major numbering, exactly a torch tensor's sizes / strides
 * / storage_offset.  dst[view index] = src[view index] for every index.
 * Transposes between the stick dim and another dim go through 64x64 tiles in
 * shared memory; everything else is moved in 16-byte units.
 * Pad lanes of the destination are zeroed where the destination view reaches
 * the end of its base's innermost dim; elements of the destination base that
 * the view does not address are left as they are.
 * Returns TS_ERR_UNSUPPORTED (and launches nothing) for a view that is not a
 * walk along single base dims, for a walk along the stick dim that neither
 * starts at a stick boundary with step 1 nor stays inside one stick, for a
 * destination with a zero stride, and for negative strides: callers then take
 * the two-pass route through ts_relayout_from_sticks / ts_relayout_to_sticks.
 * elem_bytes is 1, 2, 4 or 8 (tiled transposes: 2 only; other sizes are moved
 * element by element).  The two images must not overlap.
 */
int ts_transpose_tiles(const void* src_sticks, const int64_t* src_base, int src_base_rank,
                       const int64_t* src_strides, int64_t src_offset, void* dst_sticks,
                       const int64_t* dst_base, int dst_base_rank, const int64_t* dst_strides,
                       int64_t dst_offset, const int64_t* size, int rank, int elem_bytes,
                       void* stream);

/* Element type conversion between two stick images of one logical
 * [rows, cols] tensor, on the device: the work behind `_to_copy` with a dtype
 * change, which the reference's copy path refuses
 * (torch_spyre/csrc/spyre_mem.cpp:669-671) and its view template sends through
 * the host (codegen/templates/view.jinja2:40-46).  dtype codes: 0 = float16,
 * 1 = bfloat16, 2 = float32.  Each image has the stick width of its own type
 * (64 lanes of 2 bytes, 32 lanes of 4 bytes).  Round to nearest even; pad
 * lanes of the destination are written as zero.
 */
enum { TS_DTYPE_F16 = 0, TS_DTYPE_BF16 = 1, TS_DTYPE_F32 = 2 };
int ts_convert_sticks(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t rows,
                      int64_t cols, void* stream);

/* ---- index-driven and scan ops of the eager long tail ------------------------
 *
 * embedding (codegen/inputs/Metadata.yaml:105, "Gather"): out[t, :] =
 * weight[indices[t], :] for the tokens t of an [index_rows, index_cols] index
 * tensor.  weight is the fp16 stick image of [vocab, dim], out that of
 * [index_rows * index_cols, dim].  indices are int32 or int64 (index_bytes 4 / 8)
 * in device memory: the stick image of the index tensor when indices_are_image
 * != 0 (32 or 16 lanes per stick), else a plain array of index_rows * index_cols
 * values.  A row whose index lies outside [0, vocab) is written as zeros and
 * ts_gather_error_state() then reports 1 (it synchronises and clears the flag).
 */
int ts_embedding_rows(const void* weight, const void* indices, int index_bytes, int indices_are_image,
                      int64_t index_rows, int64_t index_cols, void* out, int64_t vocab, int64_t dim,
                      void* stream);
int ts_gather_error_state(void);

/* cumsum, which the reference computes on the host
 * (codegen/inputs/spyre_torch_ops.cpp:501-505).  fp16 in and out, fp32 running
 * sum.  ts_cumsum_rows: along the innermost (stick) dim of the stick image of
 * [rows, cols]; ts_cumsum_mid: along the middle dim of a contiguous
 * [outer][n][inner] array, which is what any other dim of a stick image is.
 */
int ts_cumsum_rows(const void* x, void* y, int64_t rows, int64_t cols, void* stream);
int ts_cumsum_mid(const void* x, void* y, int64_t outer, int64_t n, int64_t inner, void* stream);

/* upsample_nearest2d (codegen/inputs/Metadata.yaml:331,
 * "ResizeNearestNeighbor") on fp16 stick images of [planes, in_h, in_w] and
 * [planes, out_h, out_w] (planes = N * C); source index floor(dst * in / out).
 */
int ts_upsample_nearest2d(const void* x, void* y, int64_t planes, int64_t in_h, int64_t in_w,
                          int64_t out_h, int64_t out_w, void* stream);

/* SpyreTensorLayout::init (torch_spyre/csrc/spyre_tensor_impl.cpp:29-74) as a
 * plain function: fills device_size / device_strides / dim_map (rank + 1
 * entries each) for the generic stick layout of host_size; dim_order may be
 * NULL for the identity order.  Returns the number of device dims or an error.
 */
int ts_layout_init(const int64_t* host_size, int rank, int elem_bytes, const int32_t* dim_order,
                   int64_t* device_size, int64_t* device_strides, int32_t* dim_map);

/* ---- fused pointwise chain with optional row reduction --------------------
 *
 * One launch evaluates a whole fused group of fp16 pointwise ops and, if
 * asked, reduces the result along the innermost (stick) dim.  It replaces the
 * one-op-per-kernel sfp programs generate_sfp_op emits
 * (torch_spyre/_inductor/codegen/compute_ops.py:60-393, op table
 * torch_spyre/_inductor/opfuncs.py:21-84) and the eager wrappers rendered from
 * codegen/templates/base.jinja2:16-241 for the pointwise ops of
 * codegen/inputs/Metadata.yaml.
 *
 * The group is a small program for an accumulator machine working on fp16
 * values (every op result is rounded to fp16, as eager fp16 does):
 *     acc = f(acc, A [, B])
 * where A and B are operands: an input tensor, an immediate, or one of
 * TS_PW_SAVED_SLOTS saved values.
 *
 * Shapes: the iteration space is [d0, d1, d2, cols]; every tensor's stick
 * image is that of a logical tensor whose dims are either equal to the
 * iteration space's or 1 (broadcast), given as 4 int64 per tensor.
 * Full-shape outputs are written by TS_PW_STORE.  With reduce_op != 0 the
 * final acc is reduced over `cols`, multiplied by reduce_scale, and written to
 * reduce_out, which is the stick image of
 *   - [d0*d1*d2, 1]            if reduce_keepdim != 0 (one stick per row), or
 *   - [(d0*d1*d2)/reduce_inner, reduce_inner]  otherwise, reduce_inner being
 *     the extent of the innermost dim the result keeps.
 */
enum {
  TS_PW_NONE = 0, TS_PW_TENSOR = 1, TS_PW_IMM = 2, TS_PW_SAVED = 3
};
enum {
  TS_PW_LOAD = 0,  /* acc = A                          */
  TS_PW_SAVE,      /* saved[a_idx] = acc               */
  TS_PW_STORE,     /* output[a_idx] = acc              */
  TS_PW_ADD, TS_PW_SUB, TS_PW_RSUB, TS_PW_MUL, TS_PW_DIV, TS_PW_RDIV,
  TS_PW_MAX, TS_PW_MIN, TS_PW_POW,
  TS_PW_EQ, TS_PW_NE, TS_PW_LT, TS_PW_LE, TS_PW_GT, TS_PW_GE, /* acc ? A -> 1.0 / 0.0 */
  TS_PW_WHERE,     /* acc = acc != 0 ? A : B           */
  TS_PW_NEG, TS_PW_ABS, TS_PW_EXP, TS_PW_LOG, TS_PW_SQRT, TS_PW_RSQRT, TS_PW_RECIP,
  TS_PW_SIGMOID, TS_PW_TANH, TS_PW_RELU, TS_PW_SILU, TS_PW_GELU, TS_PW_GELU_TANH,
  TS_PW_SQUARE, TS_PW_LOGICAL_NOT, TS_PW_SIN, TS_PW_COS, TS_PW_ERF, TS_PW_FLOOR,
  TS_PW_CEIL, TS_PW_SIGN, TS_PW_LOG1P, TS_PW_EXPM1, TS_PW_SOFTPLUS, TS_PW_MISH,
  TS_PW_OPCOUNT
};
enum { TS_RED_NONE = 0, TS_RED_SUM = 1, TS_RED_MAX = 2, TS_RED_MIN = 3 };
#define TS_PW_MAX_INSNS 32
#define TS_PW_MAX_INPUTS 8
#define TS_PW_MAX_OUTPUTS 4
#define TS_PW_SAVED_SLOTS 4

typedef struct ts_pw_insn {
  int32_t op;
  int32_t a_kind, a_idx;
  int32_t b_kind, b_idx;
  float a_imm, b_imm;
} ts_pw_insn;

int ts_pointwise_chain(const ts_pw_insn* insns, int n_insns,
                       const void* const* inputs, const int64_t* input_shapes, int n_inputs,
                       void* const* outputs, int n_outputs,
                       const int64_t* shape /* d0, d1, d2, cols */,
                       int reduce_op, float reduce_scale, void* reduce_out,
                       int reduce_keepdim, int64_t reduce_inner, void* stream);
/* Number of chains the library holds as pre-compiled straight-line kernels (a
 * chain whose opcodes and operand selectors match one of them runs on it; any
 * other chain runs on the interpreter kernel).  No counterpart in the reference. */
int ts_pointwise_static_count(void);

/* ---- row-wise normalisations along the stick dim ---------------------------
 *
 * x and y are stick images of a logical [rows, cols] fp16 tensor (leading dims
 * flattened into rows); statistics are computed in fp32 and the result is
 * rounded to fp16 once.  cols <= TS_ROW_MAX_COLS.
 *
 * ts_softmax_rows stands in for the eager _softmax wrapper (codegen/inputs/
 * Metadata.yaml:275-277 via codegen/templates/base.jinja2:16-241) and for the
 * max/sub/exp/sum/div kernels of the compiled decomposition
 * (torch_spyre/_inductor/__init__.py:81-84).
 * ts_layernorm_rows stands in for spyre.layer_norm and its exx2 ->
 * layernormscale -> layernormnorm decomposition (torch_spyre/_inductor/
 * customops.py:74-154, decompositions.py:26-36, lowering.py:78-153); weight and
 * bias are 1-D [cols] stick images or NULL.
 * ts_rmsnorm_rows is the pow/mean/rsqrt/mul chain of an RMSNorm module fused
 * into one pass; round_before_weight != 0 rounds the normalised value to fp16
 * before the fp16 multiply by weight (module semantics), 0 rounds once.
 */
#define TS_ROW_MAX_COLS 8192
int ts_softmax_rows(const void* x, void* y, int64_t rows, int64_t cols, int log_softmax,
                    void* stream);
/* Softmax of scale * x along the stick dim under a causal mask: row r sees columns
 * 0 .. (r % period); masked positions come out as exact zeros and are not read.  x, y:
 * stick images of [rows, cols] attention scores (rows = batch * heads * period).  This is
 * the masked softmax inside scaled-dot-product attention, which the reference would get as
 * Inductor's mul / add-mask / softmax decomposition (torch_spyre/_inductor/__init__.py:81-84). */
int ts_softmax_rows_causal(const void* x, void* y, int64_t rows, int64_t cols, int64_t period,
                           float scale, void* stream);
int ts_layernorm_rows(const void* x, const void* weight, const void* bias, void* y, int64_t rows,
                      int64_t cols, float eps, void* stream);
int ts_rmsnorm_rows(const void* x, const void* weight, void* y, int64_t rows, int64_t cols,
                    float eps, int round_before_weight, void* stream);

/* ---- reductions and softmax along a non-stick dim ---------------------------
 *
 * The image is viewed as the contiguous fp16 array [outer][red][inner] with
 * inner a multiple of 8 elements (for a logical [A, red, B, cols] tensor:
 * outer = ceil(cols/64) * A, inner = B * 64).  These are the "nonstick"
 * reductions of generate_sfp_op (torch_spyre/_inductor/codegen/compute_ops.py:
 * 75-76; ops sum/max/min, torch_spyre/_inductor/opfuncs.py:26-39).
 *
 * ts_reduce_mid writes [outer][inner] = scale * reduce(x) in fp16.  When the
 * launch splits `red` over several thread blocks it needs `scratch`, a device
 * buffer of ts_reduce_mid_scratch_bytes(outer, red, inner) bytes (0 means no
 * scratch is needed and NULL may be passed).
 * ts_softmax_mid writes the softmax along red, same shape as x.
 */
int64_t ts_reduce_mid_scratch_bytes(int64_t outer, int64_t red, int64_t inner);
int ts_reduce_mid(const void* x, void* y, int64_t outer, int64_t red, int64_t inner, int reduce_op,
                  float scale, void* scratch, void* stream);
int ts_softmax_mid(const void* x, void* y, int64_t outer, int64_t red, int64_t inner,
                   int log_softmax, void* stream);

/* ts_reduce_mid for callers that cannot supply scratch memory.  This entry point has
 * no counterpart in the reference.  It exists for users of the library that own no
 * device allocator: a plug-in that only ever receives input and output pointers from
 * the application hosting it, or a caller in a latency-critical loop that must stay
 * away from cudaMalloc because an allocation can stall the whole device.
 *
 * Same arguments and result as ts_reduce_mid, minus `scratch`: when the launch splits
 * `red` over several thread blocks, the fp32 partials go to a fixed array inside the
 * library image, ts_reduce_mid_static_max_bytes() bytes (512 KiB) on every GPU that loads
 * the library, held until the process exits.  The call itself allocates nothing, on the
 * host or on the device.  A request whose partials
 * (ts_reduce_mid_scratch_bytes(outer, red, inner)) do not fit returns TS_ERR_TOO_LARGE.
 *
 * The first call on each device looks up the array's device address (with that device
 * current); make that first call outside any stream capture.  All calls on a device
 * share the one array and it keeps whatever the previous call left there; nothing in
 * it needs to start at zero, since every partial is written before it is read, but two
 * calls whose kernels overlap on the GPU (different streams) would overwrite each
 * other's partials: run them on one stream or order them with events.  The address
 * looked up by that first call is kept for the life of the process: it does not follow
 * a device whose primary context is destroyed (cudaDeviceReset) and created again, so
 * a process that resets a device must not call this entry on it afterwards. */
int ts_reduce_mid_static(const void* x, void* y, int64_t outer, int64_t red, int64_t inner,
                         int reduce_op, float scale, void* stream);
int64_t ts_reduce_mid_static_max_bytes(void);

/* ---- fp16 matmul / batched matmul on the tcgen05 tensor cores ----------------
 *
 * c[batch, M, N] = a[batch, M, K] x B (+ bias[N]), fp32 accumulation, fp16 result;
 * a, c, bias are stick images.  B is the stick image of
 *   - [batch, K, N] when b_kmajor == 0 (torch.mm / torch.bmm operand order), or
 *   - [batch, N, K] when b_kmajor != 0 (the weight of a linear layer: a x B^T);
 * with b_batched == 0 a single [K, N] / [N, K] matrix is shared by every batch
 * entry.  Pointers must be 128-byte aligned.  Stands in for spyre__mm_default,
 * spyre__bmm_default and spyre__addmm_* (codegen/inputs/spyre_torch_ops.cpp:
 * 214-452) and the compiled matmul program (torch_spyre/_inductor/lowering.py:
 * 25-47, codegen/compute_ops.py:396-824).
 *
 * ts_gemm_error_state synchronises the device and returns 1 (clearing it) if a
 * GEMM kernel gave up on one of its bounded internal waits since the last call,
 * 0 otherwise.
 */
int ts_gemm_f16(const void* a, const void* b, const void* bias, void* c, int64_t batch, int64_t M,
                int64_t N, int64_t K, int b_kmajor, int b_batched, void* stream);
int ts_gemm_error_state(void);
/* Row-parallel linear with the reduce-scatter in the GEMM's epilogue: the tensor-parallel half of
 * a linear layer whose reduction dim K is split over ranks (the sharded decoder layer of
 * tests/test_modules.py:133-211 is the reference's own goal; it has no such kernel).  This rank's
 * partial product a[M, K_local] x b (as ts_gemm_f16) is not stored: its rows belong, in `owners`
 * equal blocks of M / owners rows, to `owners` result buffers c_owner[r], each the fp16 stick image
 * of [M / owners, N] in this GPU's memory or in a peer's (a pointer obtained through CUDA IPC or
 * symmetric memory), and every tile is ADDED into its owner's buffer with 16-byte fp16x2
 * reductions at system scope as soon as it leaves the tensor cores, so the exchange over NVLink
 * runs under the rest of the GEMM.  The caller initialises each buffer (zeros, or the residual the
 * layer adds) before any rank's launch and orders the ranks around the launches (a barrier before
 * and after); the sum is formed in fp16 in arrival order, so results may differ from the
 * unsharded product in the last bits.  M / owners must be a multiple of 32, owners <= 8.
 * No TMA copy touches a peer's memory: peers are reached with plain vector reductions only. */
int ts_gemm_f16_scatter_add(const void* a, const void* b, void* const* c_owner, int owners, int64_t M,
                            int64_t N, int64_t K, int b_kmajor, void* stream);

/* The same reduce-scatter with plain peer stores instead of reductions: every tile of this rank's
 * partial product is STORED into c_owner[r], which the caller points at this rank's own slot inside
 * owner r's memory (owner r holds one [M / owners, N] image per writing rank).  Stores cross NVLink
 * as whole 128-byte sticks at link rate where fp16 reductions do not; after a barrier each owner
 * sums its slots locally with ts_sum_slots_f16, in fp32 with one rounding, so the result no longer
 * depends on arrival order.  Same argument rules as ts_gemm_f16_scatter_add.
 * Reference: none (single device, torch_spyre/__init__.py:87-89); the layer ladder of
 * tests/test_modules.py:133-211 is the goal it serves. */
int ts_gemm_f16_scatter_store(const void* a, const void* b, void* const* c_owner, int owners, int64_t M,
                              int64_t N, int64_t K, int b_kmajor, void* stream);

/* out = residual + sum of `n_slots` fp16 stick images (`slot_stride` elements apart, `n` elements
 * each, n % 8 == 0), summed in fp32 and rounded to fp16 once; `residual` may be NULL.  The local
 * half of the reduce-scatter above, and of the residual add that follows a row-parallel linear
 * (x + linear(...), tests/test_modules.py:133-211). */
int ts_sum_slots_f16(const void* slots, int n_slots, int64_t slot_stride, const void* residual, void* out,
                     int64_t n, void* stream);

/* The all-gather half of the same layer: a 2-D device-to-device copy on `stream` whose destination
 * (or source) may be a peer GPU's memory.  A rank's block of rows of a stick image is one
 * contiguous piece of `width` bytes per stick column, `height` of them, `spitch` / `dpitch` bytes
 * apart; each rank copies its block into every rank's full image.  No counterpart in the
 * reference (single device, torch_spyre/__init__.py:87-89). */
int ts_peer_copy_2d(void* dst, int64_t dpitch, const void* src, int64_t spitch, int64_t width,
                    int64_t height, void* stream);

/* Diagnostic for the give-up path of those bounded waits, without anything that could be left
 * in flight: one warp of a one-block launch waits `limit_cycles` SM clocks (clamped to
 * [1000, 10^7]) on a barrier nothing arrives on, gives up, and raises the same sticky word, so
 * ts_gemm_error_state() returns 1 once afterwards.  The reference reports runtime failures as
 * exceptions from launch_kernel (torch_spyre/csrc/module.cpp:86-109); this is the hook a test uses
 * to see the equivalent status path work end to end. */
int ts_gemm_wait_selftest(int64_t limit_cycles, void* stream);

/* ts_gemm_f16 with a residual: c = fp16(a x b [+ bias]) + residual, the sum taken in fp16 exactly
 * as a separate add of the rounded product would (residual: stick image shaped like c, may be c
 * itself's input of a skip connection, must not alias c).  Stands in for the mm + add pair of a
 * residual block (codegen/inputs/spyre_torch_ops.cpp:214-452 followed by the add wrapper of
 * codegen/templates/base.jinja2) and for addmm with a matrix-shaped bias
 * (spyre_torch_ops.cpp:380-452). */
/* A SwiGLU gate/up pair as one GEMM: c[batch, M, N_out] = silu(a x Wg^T) * (a x Wu^T), where
 * w_gate_up is the stick image of the [2*N_out, K] weight whose rows alternate in blocks of 64
 * between Wg and Wu (rows 128j..128j+63 = Wg rows 64j.., rows 128j+64..128j+127 = Wu rows 64j..).
 * N_out must be a multiple of 64.  Roundings are those of the unfused sequence (each product,
 * the silu and the multiply rounded to fp16).  Stands in for the two matmul programs, the silu
 * and the mul the reference would run for an MLP block (torch_spyre/_inductor/lowering.py:25-47,
 * codegen/compute_ops.py:60-393). */
int ts_gemm_f16_swiglu(const void* a, const void* w_gate_up, void* c, int64_t batch, int64_t M,
                       int64_t N_out, int64_t K, void* stream);

int ts_gemm_f16_residual(const void* a, const void* b, const void* bias, const void* residual,
                         void* c, int64_t batch, int64_t M, int64_t N, int64_t K, int b_kmajor,
                         int b_batched, void* stream);

/* ts_gemm_f16 with explicit image strides and an extra "heads" dim, so that the per-head
 * matmuls of attention read Q / K / V straight out of the packed [batch, seq, heads*128]
 * images and write O straight into one: for every head h and batch entry b,
 *   c_h[b] = a_h[b] x b_h[b]   (same operand conventions as ts_gemm_f16)
 * where operand X's stick column s of head h starts at X + h*X_head_stride + s*X_stick_stride
 * (elements) and holds [batch][rows][64].  A stride <= 0 selects the default of a dense
 * [batch, rows, cols] image.  Stands in for the bmm calls of an attention block
 * (codegen/inputs/spyre_torch_ops.cpp:297-377). */
int ts_gemm_f16_ex(const void* a, int64_t a_stick_stride, int64_t a_head_stride,
                   const void* b, int64_t b_stick_stride, int64_t b_head_stride,
                   const void* bias, void* c, int64_t c_stick_stride, int64_t c_head_stride,
                   int64_t heads, int64_t batch, int64_t M, int64_t N, int64_t K,
                   int b_kmajor, int b_batched, void* stream);

/* Rotary position embedding: y = x*cos + rotate_half(x)*sin per head, x / y stick images of
 * [batch*seq, heads*head_dim], cos / sin stick images of [seq, head_dim]; head_dim must be
 * 128.  One pass instead of the mul / neg / slice / cat / add programs the reference would
 * emit (torch_spyre/_inductor/opfuncs.py:49-72, codegen/data_ops.py:490-630). */
int ts_rotary_f16(const void* x, const void* cos_table, const void* sin_table, void* y,
                  int64_t batch, int64_t seq, int64_t heads, int64_t head_dim, void* stream);

/* Causal scaled-dot-product attention in one kernel: out = softmax(q k^T * scale + causal mask) v
 * per head.  q, k, v, out are the packed stick images of [batch*seq, heads*head_dim] that the
 * projection GEMMs produce / consume (head h = stick columns 2h, 2h+1); head_dim must be 128
 * (TS_ERR_UNSUPPORTED otherwise: use ts_gemm_f16_ex + ts_softmax_rows_causal); seq is free.
 * The score matrix stays on the SM.  The reference has no attention
 * kernel; this stands in for the bmm / where / _softmax / bmm programs its compiled path would
 * emit for torch.nn.functional.scaled_dot_product_attention (tests/test_modules.py:178-211 is
 * the skipped test that would exercise them).
 *
 * ts_attention_error_state: like ts_gemm_error_state, for this kernel's bounded waits. */
int ts_attention_causal_f16(const void* q, const void* k, const void* v, void* out, int64_t batch,
                            int64_t seq, int64_t heads, int64_t head_dim, float scale, void* stream);
int ts_attention_error_state(void);

#ifdef __cplusplus
}
#endif
#endif /* SPYRE_B200_H_ */
