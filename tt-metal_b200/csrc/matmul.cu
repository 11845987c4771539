// C-ABI entry points for matmul / linear and the all-gather layout helper: argument validation and
// kernel selection. Tensor-core kernels take the shapes their tiling covers; everything else goes to the
// shape-generic CUDA-core kernel, which computes the same function.
#include "common.cuh"

namespace ttb {
int32_t launch_matmul_generic(const void *a, const void *w, int w_dtype, const void *bias, void *out, int out_dtype,
                              int64_t rows, int64_t K, int64_t N, int act, int flags, cudaStream_t stream);
int32_t launch_bmm_generic(const void *a, const void *w, int w_dtype, void *out, int out_dtype, int64_t batch, int64_t M, int64_t K,
                           int64_t N, cudaStream_t stream);
bool decode_supported(int w_dtype, int64_t rows, int64_t K, int64_t N);
int64_t decode_workspace_bytes(int64_t rows, int64_t K, int64_t N, bool smem_operand);
int32_t launch_matmul_decode(const void *a, const void *w, int w_dtype, const void *bias, void *out, int out_dtype,
                             int64_t rows, int64_t K, int64_t N, int act, int flags, void *workspace,
                             int64_t workspace_bytes, bool counters_are_zero, bool compact, cudaStream_t stream,
                             const ttb_peer_gather *gather, const ttb_peer_wait_t *wait);
int32_t read_and_clear_status(cudaStream_t stream);
int32_t status_word_address(int **out);
bool prefill_supported(int w_dtype, int64_t rows, int64_t K, int64_t N);
int64_t prefill_workspace_bytes(int64_t rows, int64_t K);
int32_t launch_matmul_prefill(const void *a, const void *w, int w_dtype, const void *bias, void *out, int out_dtype, int64_t rows,
                              int64_t K, int64_t N, int act, int flags, void *workspace, int64_t workspace_bytes, int *status,
                              cudaStream_t stream);

namespace {

__global__ void gather_interleave_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, int ranks, int64_t rows,
                                         int64_t vec_per_rank_row) {
    // dst[r][g][v] = src[g][r][v], 16-byte vectors
    const int64_t total = (int64_t)ranks * rows * vec_per_rank_row;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t v = i % vec_per_rank_row;
        const int64_t g = (i / vec_per_rank_row) % ranks;
        const int64_t r = i / (vec_per_rank_row * ranks);
        dst[i] = __ldg(src + (g * rows + r) * vec_per_rank_row + v);
    }
}

int32_t validate(const void *a, int a_dtype, const void *w, int w_dtype, void *out, int out_dtype, int64_t batch, int64_t M,
                 int64_t K, int64_t N, int act) {
    if (!a || !w || !out) return fail(TTB_E_INVALID, "ttb_matmul: null tensor pointer");
    if (a_dtype != TTB_BFLOAT16) return fail(TTB_E_UNSUPPORTED, "ttb_matmul: activations must be bfloat16");
    if (w_dtype != TTB_BFLOAT8_B && w_dtype != TTB_BFLOAT4_B && w_dtype != TTB_BFLOAT16)
        return fail(TTB_E_UNSUPPORTED, "ttb_matmul: weights must be bfloat8_b, bfloat4_b or bfloat16");
    if (out_dtype != TTB_BFLOAT16 && out_dtype != TTB_FLOAT32)
        return fail(TTB_E_UNSUPPORTED, "ttb_matmul: output must be bfloat16 or float32");
    if (batch <= 0 || M <= 0 || K <= 0 || N <= 0 || M % 32 || K % 32 || N % 32)
        return fail(TTB_E_INVALID, "ttb_matmul: batch, M, K, N must be positive and M, K, N multiples of 32 (got %lld, %lld, %lld, %lld)",
                    (long long)batch, (long long)M, (long long)K, (long long)N);
    if (act < TTB_ACT_NONE || act > TTB_ACT_SILU) return fail(TTB_E_INVALID, "ttb_matmul: unknown activation %d", act);
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(TTB_E_INVALID, "ttb_matmul: tensors must be 16-byte aligned");
    return TTB_OK;
}

// Row ranges of one matmul and the tensor-core kernel that takes each: the decode kernels serve up to 256 rows, the prefill
// kernel multiples of 128 from 512 up (column counts that are multiples of 128). Row counts in between run as two decode
// launches (256 rows + the rest); a ragged count above 512 as the prefill kernel on the whole 128-row blocks plus a decode
// launch on the last 32 to 96 rows; and what the prefill kernel cannot take at all (a last column tile of fewer than 128
// columns) as decode launches over ranges of 256 rows, up to kMaxRowChunks of them. (Rows are
// contiguous in both layouts - a tile row of a tiled tensor is 32 whole rows - so a range is just an offset.)
struct RowChunk {
    int64_t row0, rows;
    bool prefill;
};
constexpr int kMaxRowChunks = 16;
int plan_rows(int w_dtype, int64_t rows, int64_t K, int64_t N, RowChunk (&out)[kMaxRowChunks]) {
    if (decode_supported(w_dtype, rows, K, N)) {
        out[0] = {0, rows, false};
        return 1;
    }
    if (prefill_supported(w_dtype, rows, K, N)) {
        out[0] = {0, rows, true};
        return 1;
    }
    if (rows > 256 && rows < 512 && decode_supported(w_dtype, 256, K, N) && decode_supported(w_dtype, rows - 256, K, N)) {
        out[0] = {0, 256, false};
        out[1] = {256, rows - 256, false};
        return 2;
    }
    const int64_t whole = rows / 128 * 128;
    if (rows > 512 && rows != whole && prefill_supported(w_dtype, whole, K, N) && decode_supported(w_dtype, rows - whole, K, N)) {
        out[0] = {0, whole, true};
        out[1] = {whole, rows - whole, false};
        return 2;
    }
    const int64_t last = rows % 256;
    if (rows >= 512 && rows <= 256 * kMaxRowChunks && decode_supported(w_dtype, 256, K, N) && (last == 0 || decode_supported(w_dtype, last, K, N))) {
        int n = 0;
        for (int64_t r0 = 0; r0 < rows; r0 += 256) out[n++] = {r0, rows - r0 < 256 ? rows - r0 : 256, false};
        return n;
    }
    return 0;
}

}  // namespace
}  // namespace ttb

using namespace ttb;

extern "C" {

int64_t ttb_matmul_workspace_bytes(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int64_t N, int32_t flags) {
    const int64_t rows = batch * M;
    if (flags & TTB_MM_FORCE_GENERIC) return 0;
    RowChunk chunks[kMaxRowChunks];
    const int n = plan_rows(w_dtype, rows, K, N, chunks);
    int64_t bytes = 0;
    for (int i = 0; i < n; ++i) {
        const int64_t b = chunks[i].prefill ? prefill_workspace_bytes(chunks[i].rows, K) : decode_workspace_bytes(chunks[i].rows, K, N, (flags & TTB_MM_DECODE_SMEM_OPERAND) != 0);
        bytes = b > bytes ? b : bytes;
    }
    return bytes;
}

/* Which kernels ttb_matmul would use: out[0] = launches (0: the shape-generic CUDA-core kernel), then per launch its rows
 * and 1 for the prefill kernel, 0 for a decode kernel - for as many launches as `out` has room for (at least two). */
int32_t ttb_matmul_plan(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int64_t N, int32_t flags, int64_t *out, int32_t out_len) {
    if (!out || out_len < 5) return fail(TTB_E_INVALID, "ttb_matmul_plan: needs room for 5 values");
    RowChunk chunks[kMaxRowChunks];
    const int n = (flags & TTB_MM_FORCE_GENERIC) ? 0 : plan_rows(w_dtype, batch * M, K, N, chunks);
    out[0] = n;
    for (int i = 0; 2 + 2 * i < out_len && i < kMaxRowChunks; ++i) {
        out[1 + 2 * i] = i < n ? chunks[i].rows : 0;
        out[2 + 2 * i] = i < n && chunks[i].prefill ? 1 : 0;
    }
    return TTB_OK;
}

int32_t ttb_matmul(const void *a, int32_t a_dtype, const void *w, int32_t w_dtype, const void *bias, void *out,
                   int32_t out_dtype, int64_t batch, int64_t M, int64_t K, int64_t N, int32_t act, int32_t flags,
                   void *workspace, int64_t workspace_bytes, void *stream) {
    if (int32_t rc = validate(a, a_dtype, w, w_dtype, out, out_dtype, batch, M, K, N, act)) return rc;
    const int64_t rows = batch * M;  // tiled [batch, M, K] with M % 32 == 0 is the same buffer as tiled [batch*M, K]
    auto s = (cudaStream_t)stream;
    RowChunk chunks[kMaxRowChunks];
    const int n = (flags & TTB_MM_FORCE_GENERIC) ? 0 : plan_rows(w_dtype, rows, K, N, chunks);
    if (n == 0) return launch_matmul_generic(a, w, w_dtype, bias, out, out_dtype, rows, K, N, act, flags, s);
    const int64_t out_elem = out_dtype == TTB_FLOAT32 ? 4 : 2;
    for (int i = 0; i < n; ++i) {
        const void *ai = static_cast<const uint8_t *>(a) + chunks[i].row0 * K * 2;
        void *oi = static_cast<uint8_t *>(out) + chunks[i].row0 * N * out_elem;
        int32_t rc;
        if (chunks[i].prefill) {
            int *status = nullptr;
            if ((rc = status_word_address(&status))) return rc;
            rc = launch_matmul_prefill(ai, w, w_dtype, bias, oi, out_dtype, chunks[i].rows, K, N, act, flags, workspace, workspace_bytes, status, s);
        } else {
            rc = launch_matmul_decode(ai, w, w_dtype, bias, oi, out_dtype, chunks[i].rows, K, N, act, flags, workspace, workspace_bytes,
                                      (flags & TTB_MM_WORKSPACE_ZEROED) != 0, /*compact=*/false, s, nullptr, nullptr);
        }
        if (rc) return rc;
    }
    return TTB_OK;
}

int32_t ttb_bmm(const void *a, int32_t a_dtype, const void *w, int32_t w_dtype, void *out, int32_t out_dtype, int64_t batch, int64_t M,
                int64_t K, int64_t N, void *stream) {
    if (int32_t rc = validate(a, a_dtype, w, w_dtype, out, out_dtype, batch, M, K, N, TTB_ACT_NONE)) return rc;
    return launch_bmm_generic(a, w, w_dtype, out, out_dtype, batch, M, K, N, (cudaStream_t)stream);
}

int32_t ttb_check_status(void *stream) { return read_and_clear_status((cudaStream_t)stream); }

int32_t ttb_gather_interleave(const void *src, void *dst, int32_t elem, int32_t ranks, int64_t rows, int64_t cols_per_rank,
                              void *stream) {
    if (!src || !dst) return fail(TTB_E_INVALID, "ttb_gather_interleave: null pointer");
    if (ranks <= 0 || rows <= 0 || cols_per_rank <= 0 || elem <= 0) return fail(TTB_E_INVALID, "ttb_gather_interleave: bad sizes");
    const int64_t row_bytes = cols_per_rank * elem;
    if (row_bytes % 16 || ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15))
        return fail(TTB_E_INVALID, "ttb_gather_interleave: per-rank rows must be a multiple of 16 bytes and pointers 16-byte aligned");
    const int64_t total = (int64_t)ranks * rows * (row_bytes / 16);
    const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
    gather_interleave_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const uint4 *)src, (uint4 *)dst, ranks, rows, row_bytes / 16);
    TTB_LAUNCH_CHECK("gather_interleave");
    return TTB_OK;
}

}  // extern "C"
