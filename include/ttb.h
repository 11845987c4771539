/*
 * libttb C ABI: the block-float weight path of TT-NN on NVIDIA B200 (sm_100a).
 *
 * Everything here is extern "C", takes plain pointers and sizes, and returns an int32 status:
 * 0 on success, a negative TTB_E_* code on failure. No call throws or aborts; a human-readable
 * description of the last failure on the calling thread is available from ttb_last_error().
 * Device pointers are caller-owned; every compute call is asynchronous on the given CUDA stream
 * (a cudaStream_t passed as void*; NULL = the default stream) unless stated otherwise.
 * Threads: one host thread drives the library at a time. The kernels' one-time set-up (function attributes, driver entry
 * points, the NCCL table, the multiprocessor count) and the launch descriptors are filled on first use without locks; callers
 * that launch from several threads serialise the calls themselves.
 *
 * Data layouts (identical to the reference's buffers, so bytes can be exchanged with it):
 *   - "tiled" = TILE_LAYOUT: tiles of 32x32 elements ordered row-major over (outer*H/32, W/32);
 *     each tile is four 16x16 row-major faces in the order top-left, top-right, bottom-left,
 *     bottom-right  (tt_metal/common/test_tiles.hpp:24-65, 124-158).
 *   - bfloat8_b tile = 1088 bytes: 64 shared-exponent bytes (byte 16*face + row) followed by 1024
 *     sign+7-bit-mantissa bytes in face order; bfloat4_b tile = 576 bytes: 64 exponent bytes followed
 *     by 512 bytes of sign+3-bit-mantissa nibbles, even element in the low nibble
 *     (tt_metal/common/blockfloat_common.hpp:174-258, tt_backend_api_types.hpp:109-132).
 *
 * The reference reaches this functionality through C++ templates and two pybind modules rather
 * than a C plugin interface; each entry point cites the reference routine it stands in for.
 */
#ifndef TTB_H_
#define TTB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------ */
#define TTB_OK 0
#define TTB_E_INVALID (-1)   /* bad argument: shape, dtype, alignment, null pointer            */
#define TTB_E_CUDA (-2)      /* a CUDA runtime call failed; ttb_last_error() holds its message */
#define TTB_E_UNSUPPORTED (-3)
#define TTB_E_WORKSPACE (-4) /* workspace missing or too small                                  */
#define TTB_E_TIMEOUT (-5)   /* a bounded device-side wait ran out (reported by ttb_check_status) */

/* ---- element types: numeric values follow tt::tt_metal::DataType
 *      (tt_eager/tensor/types.hpp:24-34) ---------------------------------------------------- */
#define TTB_BFLOAT16 0
#define TTB_FLOAT32 1
#define TTB_UINT32 2
#define TTB_BFLOAT8_B 3
#define TTB_BFLOAT4_B 4
#define TTB_UINT16 6

/* ---- fused activation after bias (ttnn.linear's `activation`, ttnn/ttnn/operations/matmul.py:59-63) */
#define TTB_ACT_NONE 0
#define TTB_ACT_RELU 1
#define TTB_ACT_GELU 2 /* erf form, the definition of the reference's torch golden (matmul.py:419-438) */
#define TTB_ACT_SILU 3

/* ---- flags for ttb_matmul ------------------------------------------------------------------ */
#define TTB_MM_A_ROW_MAJOR 1   /* activations are row-major [batch*M, K] instead of tiled        */
#define TTB_MM_OUT_ROW_MAJOR 2 /* write the result row-major (the reference's untilize_out)      */
#define TTB_MM_FORCE_GENERIC 4 /* use the shape-generic CUDA-core kernel (cross-check path)      */
#define TTB_MM_DECODE_TMEM_OPERAND 16 /* accepted for compatibility: bfloat8_b decode shapes always feed the expanded weights
                                         to the MMA through tensor memory (ldmatrix.trans + tcgen05.st) */
#define TTB_MM_DECODE_SMEM_OPERAND 128 /* bfloat8_b decode shapes: use the kernel that expands the weights into shared
                                          memory instead (the one bfloat4_b weights always use); for cross-checks */
#define TTB_MM_DETERMINISTIC 32 /* split-K partial sums are added in a fixed order (bit-reproducible results) instead
                                   of with floating-point reductions in arrival order */
#define TTB_MM_WORKSPACE_ZEROED 8 /* the first 16 MiB + 64 KiB of the workspace are zero: freshly zeroed, or
                                    last used by a completed ttb_matmul (which leaves them zero)      */
#define TTB_MM_WEIGHTS_RESIDENT 64 /* `w` was complete in device memory before the previous operation on `stream` was
                                      enqueued (weights loaded once, used many times). Decode kernels then start as a
                                      programmatic dependent of the previous kernel: they stream packed weights while it
                                      drains and wait for it before touching activations, bias, workspace or output.
                                      Takes effect together with TTB_MM_WORKSPACE_ZEROED (no memset between the kernels). */

#define TTB_MM_GATED 256 /* ttb_matmul_multi with two weights of one shape: out[0] = act(a w[0] + bias[0]) * (a w[1] + bias[1]),
                            the gated MLP's silu(x w1) * (x w3) (models/demos/mistral7b/tt/mistral_mlp.py:51-73,
                            llama2_70b/tt/llama_mlp_optimized.py:165-197) formed inside the launch; out[1] is not written.
                            Workspace: ttb_matmul_gated_workspace_bytes. Row counts of 32, 96, 160 or 224. */

const char *ttb_last_error(void);
int32_t ttb_version(void);

/* ---- device memory and copies (thin CUDA runtime wrappers so host code above this ABI needs no
 *      CUDA headers). Stand in for tt_metal Buffer allocation and EnqueueWriteBuffer /
 *      EnqueueReadBuffer (tt_eager/tensor/tensor_impl.hpp:246-269, 341-358). ------------------ */
int32_t ttb_device_count(int32_t *count);
int32_t ttb_set_device(int32_t device);
int32_t ttb_get_device(int32_t *device);
int32_t ttb_malloc(void **dev_ptr, size_t bytes);
int32_t ttb_free(void *dev_ptr);
/* Free and total device memory of the current device, as the CUDA allocator reports them (either pointer may be NULL). */
int32_t ttb_mem_info(int64_t *free_bytes, int64_t *total_bytes);
int32_t ttb_host_alloc(void **host_ptr, size_t bytes); /* pinned host memory */
int32_t ttb_host_free(void *host_ptr);
int32_t ttb_memcpy_h2d(void *dst_dev, const void *src_host, size_t bytes, void *stream);
int32_t ttb_memcpy_d2h(void *dst_host, const void *src_dev, size_t bytes, void *stream);
int32_t ttb_memcpy_d2d(void *dst_dev, const void *src_dev, size_t bytes, void *stream);
int32_t ttb_memset(void *dst_dev, int32_t value, size_t bytes, void *stream);
int32_t ttb_stream_synchronize(void *stream);
int32_t ttb_device_synchronize(void);

/* NVTX range around whatever the caller brackets with the pair (the reference marks the same spots with Tracy zones,
 * tt_metal/common/bfloat8.hpp:103,176; tt_metal/tools/profiler/op_profiler.hpp:290-312). No cost without a profiler attached. */
int32_t ttb_nvtx_push(const char *name);
int32_t ttb_nvtx_pop(void);

/* Bytes of a buffer holding outer*Hp*Wp elements of `dtype` (Hp, Wp multiples of 32 for the
 * block-float types). Mirrors compute_buffer_size (tt_eager/tensor/tensor_utils.hpp:34-47). */
int64_t ttb_buffer_bytes(int32_t dtype, int64_t outer, int64_t Hp, int64_t Wp);

/* ---- layout conversion ----------------------------------------------------------------------
 * Row-major [outer, H, W] -> tiled [outer, Hp, Wp] with zero fill of the padding, Hp/Wp = H/W
 * rounded up to 32. elem_size is 2 or 4 bytes. Replaces convert_layout(LIN_ROW_MAJOR ->
 * TILED32_4FACES) (tt_metal/common/test_tiles.hpp:178-213) and to_layout<T>
 * (tt_eager/tensor/tensor_impl.hpp:158-171, 428-499) plus pad (tensor_impl.hpp:508-677). */
int32_t ttb_tilize(const void *src_dev, void *dst_dev, int32_t elem_size, int64_t outer, int64_t H, int64_t W,
                   void *stream);
/* Tiled [outer, Hp, Wp] -> row-major [outer, H, W] (the padding is dropped). */
int32_t ttb_untilize(const void *src_dev, void *dst_dev, int32_t elem_size, int64_t outer, int64_t H, int64_t W,
                     void *stream);

/* ---- pad / unpad of row-major tensors -----------------------------------------------------------
 * ttb_pad: dst[out_shape] = pad value everywhere except the box starting at `start`, which receives src[in_shape]
 * (four dimensions, row-major, elem_size 2 or 4 bytes; pad_bits holds the pad value's bit pattern in its low bits).
 * ttb_unpad: dst = src[start[0]..end[0], ..., start[3]..end[3]] (both ends inclusive, as in the reference).
 * Replace pad<T> / unpad<T> (tt_eager/tensor/tensor_impl.hpp:508-677), which run on host vectors. */
int32_t ttb_pad(const void *src_dev, void *dst_dev, int32_t elem_size, const int64_t *in_shape, const int64_t *out_shape,
                const int64_t *start, uint32_t pad_bits, void *stream);
int32_t ttb_unpad(const void *src_dev, void *dst_dev, int32_t elem_size, const int64_t *in_shape, const int64_t *start,
                  const int64_t *end, void *stream);

/* Elementwise product of two bfloat16 buffers of `count` elements (any layout, as long as both share it): the unfused form of
 * the gated MLP's multiply, tt_lib.tensor.mul in models/demos/llama2_70b/tt/llama_mlp_optimized.py:191-197. */
int32_t ttb_mul_bf16(const void *a_dev, const void *b_dev, void *out_dev, int64_t count, void *stream);

/* ---- block-float pack / unpack --------------------------------------------------------------
 * ttb_pack_bfp: src (TTB_FLOAT32 or TTB_BFLOAT16) -> packed tiles of `fmt` (TTB_BFLOAT8_B or
 * TTB_BFLOAT4_B). With src_row_major != 0 the source is row-major [outer, H, W] and tilize, zero
 * padding to 32 and packing happen in one pass; otherwise the source already is tiled
 * [outer, H, W] (H, W multiples of 32) and is consumed sequentially. Bit-exact with
 * pack_fp32_vec_as_bfp8_tiles / pack_fp32_vec_as_bfp4_tiles (tt_metal/common/bfloat8.hpp:102-173,
 * bfloat4.hpp:23-25, blockfloat_common.hpp:19-258).
 * With two_pass != 0 every group of 16 values goes through pack -> unpack -> pack, which is what
 * ttnn.from_torch does on the host (pytensor.cpp:145-160 then tensor_impl.cpp:179-197); the bytes
 * differ from the single pass only for non-finite or denormal inputs. */
int32_t ttb_pack_bfp(const void *src_dev, int32_t src_dtype, void *dst_dev, int32_t fmt, int64_t outer, int64_t H,
                     int64_t W, int32_t src_row_major, int32_t two_pass, void *stream);

/* ttb_unpack_bfp: packed tiles of `fmt` holding a tiled [outer, Hp, Wp] tensor -> dst
 * (TTB_FLOAT32 or TTB_BFLOAT16; both exact, the unpacked values have at most 8 significant bits),
 * row-major [outer, H, W] without the padding when dst_row_major != 0, else tiled (H, W multiples
 * of 32). Bit-exact with unpack_bfp8_tiles_into_float_vec / unpack_bfp4_tiles_into_float_vec
 * (bfloat8.hpp:175-265, bfloat4.hpp:33-164), including the unclamped exponent arithmetic.
 * With two_pass != 0 every group of 16 values goes through unpack -> pack -> unpack as
 * ttnn.to_torch does (tensor_impl.cpp:179-197, pytensor.cpp:382-393). */
int32_t ttb_unpack_bfp(const void *src_dev, int32_t fmt, void *dst_dev, int32_t dst_dtype, int64_t outer, int64_t H,
                       int64_t W, int32_t dst_row_major, int32_t two_pass, void *stream);

/* ---- matmul / linear --------------------------------------------------------------------------
 * out[b, M, N] = act( a[b, M, K] x w[K, N] + bias[N] ), fp32 accumulation.
 *   a:    TTB_BFLOAT16, tiled (or row-major with TTB_MM_A_ROW_MAJOR); M, K multiples of 32.
 *   w:    TTB_BFLOAT8_B, TTB_BFLOAT4_B or TTB_BFLOAT16, tiled [K, N], shared by every batch entry.
 *   bias: NULL, or TTB_BFLOAT16 tiled [32, N] whose first row is used (the reference's
 *         [1,1,32,N] bias tile row, tt_eager/tt_dnn/op_library/bmm/bmm_op.cpp:859-863).
 *   out:  TTB_BFLOAT16 or TTB_FLOAT32, tiled (or row-major with TTB_MM_OUT_ROW_MAJOR).
 * Block-float weights are expanded to bf16 in shared memory (exact) and multiplied on the tcgen05
 * tensor cores; shapes outside the tensor-core kernels' tiling use a CUDA-core kernel with the same
 * arithmetic. Stands in for tt::operations::primary::matmul and the multi-core-reuse program
 * factories (bmm_op.hpp:284-346, bmm_op.cpp:828-1303, and the multi_core_reuse program factories
 * beside them). `workspace` is device scratch of at least ttb_matmul_workspace_bytes() bytes (may be NULL when
 * that is 0); it is only touched between launch and completion of this call on `stream`. Its head holds
 * per-output-tile arrival counters that must be zero when the kernel starts: ttb_matmul clears them with a
 * memset on `stream` unless TTB_MM_WORKSPACE_ZEROED is given. */
int64_t ttb_matmul_workspace_bytes(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int64_t N, int32_t flags);
/* Which kernels ttb_matmul uses for a shape (no GPU needed): out[0] = launches (0: the shape-generic CUDA-core kernel;
 * else tensor-core launches over consecutive row ranges), then per launch its row count and 1 for the prefill kernel, 0
 * for a decode kernel - for as many launches as `out` has room for (out_len >= 5). Decode kernels take up to 256 rows and
 * any N that is a multiple of 32 (blocks of two tile rows when the row count is a multiple of 64 and N a multiple of 128,
 * else of one); the prefill kernel multiples of 128 rows from 512 up with N a multiple of 128; other row counts are served
 * as two ranges, and large row counts with an N the prefill kernel does not take as up to 16 decode launches of 256 rows. */
int32_t ttb_matmul_plan(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int64_t N, int32_t flags, int64_t *out, int32_t out_len);
int32_t ttb_matmul(const void *a_dev, int32_t a_dtype, const void *w_dev, int32_t w_dtype, const void *bias_dev,
                   void *out_dev, int32_t out_dtype, int64_t batch, int64_t M, int64_t K, int64_t N,
                   int32_t activation, int32_t flags, void *workspace_dev, int64_t workspace_bytes, void *stream);

/* Batched matmul with a batched second operand: out[b, M, N] = a[b, M, K] x w[b, K, N] for b < batch, every operand tiled,
 * `a` bfloat16, `w` bfloat8_b / bfloat4_b / bfloat16 (one packed [K, N] matrix after the other), fp32 accumulation, bfloat16 or
 * float32 output. Stands in for tt::tt_metal::bmm and the batched form of tt::operations::primary::matmul
 * (tt_eager/tt_dnn/op_library/bmm/bmm_op.hpp:388-456, bmm_op.cpp:518-626; attention's Q K^T and P V products,
 * tests/tt_eager/python_api_testing/unit_testing/misc/test_matmul.py:204-320). Runs on the CUDA cores. */
int32_t ttb_bmm(const void *a_dev, int32_t a_dtype, const void *w_dev, int32_t w_dtype, void *out_dev, int32_t out_dtype, int64_t batch,
                int64_t M, int64_t K, int64_t N, void *stream);

/* Decode matmul for callers that cannot allocate device memory.
 * This entry point has no counterpart in the reference. It computes exactly what ttb_matmul computes for the decode
 * shapes (bfloat16 activations of at most 256 rows in total, bfloat8_b / bfloat4_b weights, N a multiple of 128), but
 * takes no workspace: the scratch the split-K reduction needs is a fixed array inside the library's device image
 * (16 MiB + 64 KiB, resident on every GPU that loads the library, for the life of the process). It is meant for
 * code that runs where cudaMalloc is off limits - inside a serving loop that has handed all device memory to its own
 * pool, in a callback of another runtime, or in any path that must not trigger the implicit synchronisation
 * of an allocation. The call itself performs no cudaMalloc / cudaFree and uses no allocating library routine.
 *   - Shapes whose reduction needs more scratch than the array holds are refused with TTB_E_WORKSPACE, other
 *     shapes than the decode ones with TTB_E_UNSUPPORTED; both point to ttb_matmul.
 *   - The first call on each device looks up the array's device address (and sets the kernel's shared-memory
 *     limit); make that first call outside any stream capture.
 *   - All calls share the one array, which keeps the previous call's contents; the part that must start at zero is
 *     cleared on `stream` by each call. Two calls that overlap on the GPU (different streams, no dependency) race on
 *     it: serialise them.
 * `flags` accepts TTB_MM_A_ROW_MAJOR and TTB_MM_OUT_ROW_MAJOR. */
/* Scratch a shape would need from the built-in array (it holds 16 MiB + 64 KiB); -1 for shapes that are not decode shapes. */
int64_t ttb_matmul_decode_static_scratch_bytes(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int64_t N);
int32_t ttb_matmul_decode_static(const void *a_dev, int32_t a_dtype, const void *w_dev, int32_t w_dtype, const void *bias_dev,
                                 void *out_dev, int32_t out_dtype, int64_t batch, int64_t M, int64_t K, int64_t N,
                                 int32_t activation, int32_t flags, void *stream);

/* Reads (and clears) the device-side status word that kernels with bounded waits set when a wait
 * ran out. Synchronises `stream`. Returns TTB_OK or TTB_E_TIMEOUT. After TTB_E_TIMEOUT the matmul that gave up has
 * produced no valid output and may have left arrival counters and accumulation tiles of its workspace non-zero:
 * clear the workspace head (or drop TTB_MM_WORKSPACE_ZEROED for the next call) before reusing it. */
int32_t ttb_check_status(void *stream);
/* Limit of every bounded device-side wait (waits for peers' data, and the pipeline barriers inside the matmul kernels,
 * which get twice this plus a margin), in SM clock cycles, for launches made after the call; 0 restores the built-in
 * defaults (about ten seconds for peers, one second for barriers). Process-wide, not synchronised with concurrent
 * launches from other host threads. Stands in for the host-side timeouts of the reference's device polling loops
 * (a hung Tensix core is detected by the watcher / a dispatch timeout, tt_metal/impl/debug/watcher_server.cpp). */
int32_t ttb_set_wait_limit_cycles(int64_t cycles);

/* ---- all-gather helper ------------------------------------------------------------------------
 * After a rank-major gather of G slices [rows, cols_per_rank] (what an NCCL all-gather leaves),
 * interleave them into row-major [rows, G*cols_per_rank]. Not needed for tiled tensors whose row
 * count is one tile (32): there the rank-major gather already is the tiled [32, G*cols] tensor.
 * Stands in for the concat-along-dim semantics of AllGather
 * (tt_eager/tt_dnn/op_library/all_gather/all_gather_op.cpp:18-104). */
int32_t ttb_gather_interleave(const void *src_dev, void *dst_dev, int32_t elem_size, int32_t ranks, int64_t rows,
                              int64_t cols_per_rank, void *stream);

/* ---- communicator (one process per GPU) ---------------------------------------------------------
 * NCCL over NVLink behind plain C, for the general form of ttnn.all_gather. Replaces the ring set-up and the AllGather op of
 * the reference (tt_eager/tt_dnn/op_library/all_gather/all_gather_op.cpp:18-104, ttnn/ttnn/operations/ccl.py:26-39).
 * Rank 0 makes a unique id (TTB_COMM_ID_BYTES bytes) and hands it to the other ranks by any means; every rank then calls
 * ttb_comm_init with its device current. Initialisation is non-blocking inside: the call polls the communicator's state and
 * gives up after timeout_ms of host time (a peer that never joins) with TTB_E_TIMEOUT, having aborted the half-built
 * communicator; timeout_ms < 0 waits without limit. ttb_comm_check polls a live communicator for an asynchronous error
 * (TTB_E_CUDA) or for work still being enqueued (TTB_E_TIMEOUT after timeout_ms); after either, ttb_comm_abort is the only
 * valid call. ttb_all_gather enqueues out[r * bytes_per_rank ...] = rank r's src on `stream` (rank-major concatenation of
 * byte runs; tiled shards of one tile row and row-major single-row shards already are the gathered tensor, others go
 * through ttb_gather_interleave). NCCL is loaded at first use (libnccl.so.2); where it is absent these calls return
 * TTB_E_UNSUPPORTED and everything else works. */
#define TTB_COMM_ID_BYTES 128
int32_t ttb_comm_unique_id(void *id);
int32_t ttb_comm_init(void **comm, int32_t ranks, int32_t rank, const void *unique_id, int64_t timeout_ms);
int32_t ttb_comm_check(void *comm, int64_t timeout_ms);
int32_t ttb_all_gather(void *comm, const void *src_dev, void *dst_dev, int64_t bytes_per_rank, void *stream);
int32_t ttb_comm_abort(void *comm);   /* tears the communicator down without waiting for its peers; frees `comm` */
int32_t ttb_comm_destroy(void *comm); /* orderly release after all work has completed; frees `comm` */
/* The calls above reach the collective library through this table (result codes: 0 success, 7 still in progress, others
 * errors). Passing a table replaces the library - tests use it to produce a peer that never joins or an asynchronous
 * error on the host, with no GPU involved; NULL restores the real library. init_rank_config(comm, ranks, id, rank, user). */
typedef struct ttb_comm_backend {
    int (*get_unique_id)(void *id);
    int (*init_rank_config)(void **comm, int ranks, const void *id, int rank, void *user);
    int (*get_async_error)(void *comm, int *state);
    int (*all_gather)(const void *src, void *dst, size_t count, int dtype, void *comm, void *stream);
    int (*abort)(void *comm);
    int (*destroy)(void *comm);
    const char *(*error_string)(int code);
    void *user;
} ttb_comm_backend;
int32_t ttb_comm_set_backend(const ttb_comm_backend *backend);

/* ---- matmul with the all-gather in its epilogue (tensor-parallel decode) -------------------------
 * One process per GPU. Every rank computes its column slice out[:, rank*N : (rank+1)*N] of a gathered
 * [batch*M, ranks*N] bfloat16 tiled tensor and stores each finished tile into its own copy and, over NVLink with plain
 * peer stores, into every other rank's copy; no separate collective runs. Replaces ttnn.all_gather(ttnn.linear(x, w),
 * dim=-1) (ttnn/ttnn/operations/ccl.py:26-39, tt_eager/tt_dnn/op_library/all_gather/all_gather_op.cpp:18-104,
 * column-sharded weights as models/demos/llama2_70b/tt/llama_mlp_optimized.py:100-103).
 *
 * A gather point is a pair of 32-bit counters on every rank, both starting at zero: `arrived`, to which every rank adds
 * one per finished output tile (over NVLink), and `expected`, the running total of arrivals that the owning rank's own
 * gathering launches announce (ranks x tiles per launch; all ranks launch the same shapes). The gathered copy on a rank is
 * complete when arrived >= expected. A later ttb_matmul_peer on the same stream that passes the gather point as `wait`
 * holds its activation loads until then (its weight streaming is not held); any other consumer first runs ttb_peer_wait on
 * the stream. Waits are bounded (about ten seconds) and end in TTB_E_TIMEOUT through ttb_check_status instead of hanging.
 * Rules the caller keeps: all ranks issue the same sequence of gathering launches; consecutive gathering launches on a
 * stream use different gather points and different output buffers (two of each, alternating, suffice), and every gathering
 * launch is waited for (by a consuming ttb_matmul_peer or by ttb_peer_wait) no later than in the next gathering launch on
 * that stream, which keeps any rank from running more than one gather ahead of another;
 * peer pointers come from ttb_ipc_open on handles made by ttb_ipc_export in the owning process. Decode shapes only
 * (as ttb_matmul_decode_static), bfloat16 tiled output; workspace as ttb_matmul (ttb_matmul_peer_workspace_bytes). */
#define TTB_MAX_RANKS 8
#define TTB_MAX_GROUP 4 /* weights per ttb_matmul_multi launch */
typedef struct ttb_peer_gather {
    int32_t ranks;                     /* 2..TTB_MAX_RANKS */
    int32_t rank;                      /* this process's position */
    void *out[TTB_MAX_RANKS];          /* the gathered tensor on every rank as mapped into this process; out[rank] is local */
    uint32_t *arrived[TTB_MAX_RANKS];  /* the gather point's arrival counter on every rank; arrived[rank] is local */
    uint32_t *expected;                /* the gather point's local expected-arrivals counter */
} ttb_peer_gather;
typedef struct ttb_peer_wait_t {
    const uint32_t *arrived;           /* local arrival counter of the gather point that produced the activations */
    const uint32_t *expected;          /* its local expected-arrivals counter */
} ttb_peer_wait_t;
int64_t ttb_matmul_peer_workspace_bytes(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int64_t N);
/* `gather` and `wait` may each be NULL: without `gather` the result is an ordinary local matmul into out_dev (then
 * `out_dev` is used, otherwise gather->out[rank]); without `wait` the activations are assumed complete. */
int32_t ttb_matmul_peer(const void *a_dev, int32_t a_dtype, const void *w_dev, int32_t w_dtype, const void *bias_dev,
                        void *out_dev, int32_t out_dtype, int64_t batch, int64_t M, int64_t K, int64_t N,
                        int32_t activation, int32_t flags, void *workspace_dev, int64_t workspace_bytes,
                        const ttb_peer_gather *gather, const ttb_peer_wait_t *wait, void *stream);
/* Several weights that multiply the same activation, in one launch: out[j] = act(a x w[j] + bias[j]), j < count <=
 * TTB_MAX_GROUP, every weight [K, N[j]] in the same block-float format. What the reference's models issue as separate
 * matmuls on one input - the q / k / v projections (models/demos/mistral7b/tt/mistral_attention.py:72-99, which fuses them
 * by concatenating the weights) and the w1 / w3 projections of the gated MLP (mistral_mlp.py:51-73,
 * llama2_70b/tt/llama_mlp_optimized.py:165-193) - becomes one pass of one persistent kernel over all their tiles; the
 * weights stay separate tensors. Decode shapes only. `bias` may be NULL or hold NULL entries. `gather` (may be NULL)
 * applies to weight 0 only: its result goes to gather->out[...] on every rank and out[0] is ignored; `wait` as in
 * ttb_matmul_peer. Results agree with `count` calls of ttb_matmul up to the order in which fp32 partial sums are added. */
int64_t ttb_matmul_multi_workspace_bytes(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int32_t count, const int64_t *N);
int64_t ttb_matmul_gated_workspace_bytes(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int64_t N);
int32_t ttb_matmul_multi(const void *a_dev, int32_t a_dtype, int32_t count, const void *const *w_dev, int32_t w_dtype,
                         const void *const *bias_dev, void *const *out_dev, int32_t out_dtype, int64_t batch, int64_t M,
                         int64_t K, const int64_t *N, int32_t activation, int32_t flags, void *workspace_dev,
                         int64_t workspace_bytes, const ttb_peer_gather *gather, const ttb_peer_wait_t *wait, void *stream);
/* Several ttb_matmul_multi calls as the stages of ONE launch. The persistent blocks walk the stages in order without
 * meeting in between: the weight stream of stage s + 1 starts while stage s drains, and a stage whose activation is an
 * earlier stage's output (`input_from`) or a gathered tensor (`wait`) holds back only its activation copies until that
 * is complete. What the reference's decode MLP issues as matmul, matmul, multiply, matmul on one device
 * (models/demos/llama2_70b/tt/llama_mlp_optimized.py:165-218, models/demos/mistral7b/tt/mistral_mlp.py:51-73) becomes
 * two stages: the gated pair, then the down projection. Row counts that are odd multiples of 32 (one tile row per
 * block); all weights of the launch in one block-float format. Results agree with the separate calls up to the order in
 * which fp32 partial sums over K are added (and repeat exactly from launch to launch under TTB_MM_DETERMINISTIC). */
typedef struct ttb_matmul_stage {
    const void *a;                     /* activation [batch * M, K], bf16 (for input_from >= 0: that stage's out[0]) */
    int32_t count;                     /* weights of the stage, 1..TTB_MAX_GROUP */
    const void *w[TTB_MAX_GROUP];
    const void *bias[TTB_MAX_GROUP];   /* entries may be NULL */
    void *out[TTB_MAX_GROUP];
    int32_t out_dtype;
    int64_t K;
    int64_t N[TTB_MAX_GROUP];
    int32_t activation;
    int32_t flags;                     /* TTB_MM_A_ROW_MAJOR | TTB_MM_OUT_ROW_MAJOR | TTB_MM_DETERMINISTIC | TTB_MM_GATED */
    const ttb_peer_gather *gather;     /* as in ttb_matmul_multi; may be NULL */
    const ttb_peer_wait_t *wait;       /* as in ttb_matmul_multi; may be NULL */
    int32_t input_from;                /* index of the earlier stage that writes `a`, or -1 */
} ttb_matmul_stage;
#define TTB_MAX_STAGES 4
int64_t ttb_matmul_sequence_workspace_bytes(int32_t w_dtype, int64_t batch, int64_t M, const ttb_matmul_stage *stages, int32_t count);
/* `flags`: TTB_MM_WORKSPACE_ZEROED | TTB_MM_WEIGHTS_RESIDENT for the launch as a whole. */
int32_t ttb_matmul_sequence(const ttb_matmul_stage *stages, int32_t count, int32_t a_dtype, int32_t w_dtype, int64_t batch, int64_t M,
                            int32_t flags, void *workspace_dev, int64_t workspace_bytes, void *stream);
/* The work decomposition ttb_matmul / ttb_matmul_multi use for a decode shape (no GPU needed). out[0..9] = rows per block,
 * tiles (128 columns x rows per block) in the launch, persistent blocks, K pieces per tile (1 = whole tiles round by round
 * plus a streamed remainder), K blocks (of 32) per piece, rounds of whole tiles / pieces, first tile of the streamed
 * remainder (or the piece count), units of 8 K blocks in the streamed remainder, units per tile, partial-sum slots. */
int32_t ttb_matmul_decode_plan(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int32_t count, const int64_t *N,
                               int32_t *out, int32_t out_len);
/* Holds `stream` until the gather point's current use is complete on this rank (bounded). */
int32_t ttb_peer_wait(const ttb_peer_wait_t *wait, void *stream);
/* CUDA IPC plumbing for the peer pointers: `handle` is a 64-byte buffer. `ptr_dev` must be the start of an allocation
 * made by ttb_malloc. ttb_ipc_open maps a peer's allocation into this process (enabling peer access). */
#define TTB_IPC_HANDLE_BYTES 64
int32_t ttb_ipc_export(void *ptr_dev, void *handle);
int32_t ttb_ipc_open(const void *handle, void **ptr_dev);
int32_t ttb_ipc_close(void *ptr_dev);

#ifdef __cplusplus
}
#endif
#endif /* TTB_H_ */
