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
int64_t decode_workspace_bytes(int64_t rows, int64_t K, int64_t N);
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

}  // namespace
}  // namespace ttb

using namespace ttb;

extern "C" {

int64_t ttb_matmul_workspace_bytes(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int64_t N, int32_t flags) {
    const int64_t rows = batch * M;
    if (flags & TTB_MM_FORCE_GENERIC) return 0;
    if (decode_supported(w_dtype, rows, K, N)) return decode_workspace_bytes(rows, K, N);
    if (prefill_supported(w_dtype, rows, K, N)) return prefill_workspace_bytes(rows, K);
    return 0;
}

int32_t ttb_matmul(const void *a, int32_t a_dtype, const void *w, int32_t w_dtype, const void *bias, void *out,
                   int32_t out_dtype, int64_t batch, int64_t M, int64_t K, int64_t N, int32_t act, int32_t flags,
                   void *workspace, int64_t workspace_bytes, void *stream) {
    if (int32_t rc = validate(a, a_dtype, w, w_dtype, out, out_dtype, batch, M, K, N, act)) return rc;
    const int64_t rows = batch * M;  // tiled [batch, M, K] with M % 32 == 0 is the same buffer as tiled [batch*M, K]
    auto s = (cudaStream_t)stream;
    if (!(flags & TTB_MM_FORCE_GENERIC) && decode_supported(w_dtype, rows, K, N))
        return launch_matmul_decode(a, w, w_dtype, bias, out, out_dtype, rows, K, N, act, flags, workspace, workspace_bytes,
                                    (flags & TTB_MM_WORKSPACE_ZEROED) != 0, /*compact=*/false, s, nullptr, nullptr);
    if (!(flags & TTB_MM_FORCE_GENERIC) && prefill_supported(w_dtype, rows, K, N)) {
        int *status = nullptr;
        if (int32_t rc = status_word_address(&status)) return rc;
        return launch_matmul_prefill(a, w, w_dtype, bias, out, out_dtype, rows, K, N, act, flags, workspace, workspace_bytes, status, s);
    }
    return launch_matmul_generic(a, w, w_dtype, bias, out, out_dtype, rows, K, N, act, flags, s);
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
