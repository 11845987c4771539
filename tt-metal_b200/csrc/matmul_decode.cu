// Host side of the decode (small row count) matmuls: planning of the streamed decomposition, workspace layout, dispatch
// to the kernels (matmul_decode_stream.cu; matmul_decode_tmem.cu for 128-row blocks of bfloat8_b), the allocation-free
// entry point, the entry point whose epilogue is the all-gather, and the device status word of the bounded waits.
#include <type_traits>

#include "decode_smem.cuh"

namespace ttb {

__device__ int g_status_word = 0;

// Limit of the bounded device-side waits in SM clocks; 0 = each wait's built-in default. Read at launch time.
static long long g_wait_limit_cycles = 0;
long long wait_limit_cycles() { return g_wait_limit_cycles; }

using namespace decode_smem;

// The head of the workspace holds one arrival counter per output tile; the partial sums follow.
static constexpr int64_t kCounterBytes = 65536;
// Workspace layout: [arrival counters, 64 KiB][accumulate-mode tiles, 16 MiB, zero between launches][ordered-mode
// partials / other scratch]. The compact layout (built-in scratch of the allocation-free entry point) has no middle part.
static constexpr int64_t kAccumBytes = 16 << 20;

int32_t launch_decode_tmem(const DecodeArgs *stages, int n, int fmt, int nb, int *sync, bool overlap, cudaStream_t stream);
// The tail of the counter region belongs to the launch as a whole (matmul_decode_tmem.cu: blocks that have finished, tiles
// each stage has stored); the per-tile counters stay below it.
static constexpr int kSyncInts = 16;
static constexpr int kSyncInt0 = (int)(65536 / 4) - kSyncInts;

// Device address of the status word on the current device (looked up once per device).
int32_t status_word_address(int **out) {
    static int *cached[64] = {};
    int dev = 0;
    TTB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 64 || !cached[dev % 64]) {
        void *ptr = nullptr;
        TTB_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_status_word));
        if (dev >= 64) { *out = (int *)ptr; return TTB_OK; }
        cached[dev] = (int *)ptr;
    }
    *out = cached[dev];
    return TTB_OK;
}

// Rows per block. The tensor-memory kernel takes one or two tile rows (32 or 64 rows); the shared-memory-operand kernel (on
// request) the largest of 128 / 64 / 32 that divides the row count. A weight whose last column tile holds fewer than 128
// columns (`ragged`) is served by blocks of one tile row only.
static int decode_rows_per_block(int64_t rows, bool smem_operand, bool ragged) {
    if (ragged) return 32;
    if (smem_operand) return rows % 128 == 0 ? 128 : rows % 64 == 0 ? 64 : 32;
    return rows % 64 == 0 ? 64 : 32;
}

// 128-column tiles of a weight of N columns. The last one may hold 32, 64 or 96 columns (its missing packed tiles read as
// zeros and the epilogue stores no column beyond N).
static int tiles128(int64_t N) { return (int)((N + BN - 1) / BN); }
static bool columns_ok(int64_t N) { return N > 0 && N % 32 == 0; }
static bool any_ragged(int nprob, const int64_t *N) {
    for (int j = 0; j < nprob; ++j)
        if (N[j] % BN) return true;
    return false;
}

bool decode_supported(int w_dtype, int64_t rows, int64_t K, int64_t N) {
    return (w_dtype == TTB_BFLOAT8_B || w_dtype == TTB_BFLOAT4_B) && rows > 0 && rows <= 256 && rows % 32 == 0 &&
           K % BK == 0 && columns_ok(N) && tiles128(N) * (rows / 32) <= kSyncInt0;
}

// ---- streamed decomposition (matmul_decode_stream.cu) ----------------------------------------------------------------
int32_t launch_decode_stream(const DecodeArgs &p, int fmt, int nb, bool overlap, cudaStream_t stream);

struct StreamPlan {
    int nb, rchunks, tiles_row, tiles_total, grid, gran, upt;
    int pieces, kbps;       // pieces decomposition: parts per tile (1 = not used) and K-blocks per part
    int waves, rem_tile0;   // rounds of whole tiles (or pieces); first tile of the remainder that is streamed (or the piece count)
    long long units;        // units of the streamed remainder
    int slots;              // partial-sum slots
    bool shared_tiles;      // some tile's K range is shared by several blocks: scratch needed
};
// One persistent block per multiprocessor of the current device (read once per process; 148, a B200's count, where no device
// can be asked - the plan and workspace queries also work without a GPU).
static int stream_blocks() {
    static int cached = 0;
    if (cached == 0) {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0)
            cached = sms;
        else
            cached = 148;
        (void)cudaGetLastError();
    }
    return cached;
}
static constexpr int kStreamGran = 8;   // K-blocks per unit: no block gets a piece of a tile shorter than this

// Picks the cheaper of two decompositions by a small cost model in units of one K-block's streaming time (~0.083 us per
// block of the tensor-memory kernel):
//  * pieces: every tile cut into s equal parts along K, taken round by round - cost rounds * (K-blocks per part, rounded
//    up to whole groups of four, + 6, + 20 when s > 1) + 45 once when s > 1 for the partial-sum exchange of the last round
//    (~4-5 us from the last reduction to the finished tile, nearly independent of s);
//  * whole tiles round by round, the tiles left after the last full round streamed evenly over all blocks (1.15 per
//    K-block: all multiprocessors pull on HBM) - each block then has up to two shared segments, ~45 / ~80 for their
//    exchanges and the pipeline bubbles around them.
// Both pay ~50 once for filling and draining the pipeline. Calibrated on B200 timings of the Llama-70B shapes and their
// 2-, 4- and 8-way column shards (sweeps over s and both forms per shape).
static StreamPlan stream_plan(int64_t rows, int64_t K, int nprob, const int64_t *N, bool smem_operand = false) {
    const int kStreamBlocks = stream_blocks();
    StreamPlan sp;
    sp.nb = decode_rows_per_block(rows, smem_operand, any_ragged(nprob, N));
    sp.rchunks = (int)(rows / sp.nb);
    sp.tiles_row = 0;
    for (int j = 0; j < nprob; ++j) sp.tiles_row += tiles128(N[j]);
    sp.tiles_total = sp.tiles_row * sp.rchunks;
    const int nkb = (int)(K / BK);
    sp.gran = kStreamGran;
    sp.upt = (nkb + sp.gran - 1) / sp.gran;
    const int T = sp.tiles_total;
    // pieces
    int best_s = 1;
    double best_cost = 1e30;
    for (int s = 1; s <= 32 && s <= nkb; ++s) {
        const int kbps = (nkb + s - 1) / s;
        if ((nkb + kbps - 1) / kbps != s) continue;
        if (s > 1 && kbps < 8) break;
        const int rounds = (T * s + kStreamBlocks - 1) / kStreamBlocks;
        const double cost = rounds * ((kbps + 3) / 4 * 4 + 6.0 + (s > 1 ? 20.0 : 0.0)) + (s > 1 ? 45.0 : 0.0);
        if (cost < best_cost) { best_cost = cost; best_s = s; }
    }
    // whole tiles + streamed remainder
    const int full = T / kStreamBlocks, rem = T % kStreamBlocks;
    double stream_cost = 1e30;
    if (rem > 0 && (long long)rem * sp.upt >= 2) {
        const double share = (double)rem * nkb / kStreamBlocks;
        stream_cost = full * (nkb + 6.0) + 1.15 * share + (full > 0 ? 45.0 : 80.0);   // after whole tiles a block has one shared segment, else two
    }
    if (stream_cost < best_cost) {
        sp.pieces = 1; sp.kbps = nkb;
        sp.waves = full;
        sp.rem_tile0 = full * kStreamBlocks;
        sp.units = (long long)rem * sp.upt;
        sp.grid = full > 0 ? kStreamBlocks : (int)(sp.units < kStreamBlocks ? sp.units : kStreamBlocks);
        sp.slots = rem + sp.grid;
        sp.shared_tiles = false;
        const long long q = sp.units / sp.grid, r = sp.units % sp.grid;
        for (int b = 1; b < sp.grid; ++b)
            if ((b * q + (b < r ? b : r)) % sp.upt != 0) sp.shared_tiles = true;
    } else {
        sp.pieces = best_s; sp.kbps = (nkb + best_s - 1) / best_s;
        const int npieces = T * best_s;
        sp.waves = (npieces + kStreamBlocks - 1) / kStreamBlocks;
        sp.rem_tile0 = npieces;
        sp.units = 0;
        sp.grid = npieces < kStreamBlocks ? npieces : kStreamBlocks;
        sp.slots = best_s > 1 ? npieces : 0;
        sp.shared_tiles = best_s > 1;
    }
    return sp;
}

bool decode_supported_multi(int w_dtype, int64_t rows, int64_t K, int nprob, const int64_t *N) {
    if (!(w_dtype == TTB_BFLOAT8_B || w_dtype == TTB_BFLOAT4_B) || rows <= 0 || rows > 256 || rows % 32 || K <= 0 || K % BK) return false;
    if (nprob < 1 || nprob > TTB_MAX_GROUP) return false;
    int64_t tiles = 0;
    for (int j = 0; j < nprob; ++j) {
        if (!columns_ok(N[j])) return false;
        tiles += tiles128(N[j]);
    }
    return tiles * (rows / 32) <= kSyncInt0;
}

// Accumulate mode needs rows * (sum of N) fp32 inside the fixed 16 MiB region; larger outputs use ordered mode.
static bool stream_accumulate_ok(int64_t rows, int nprob, const int64_t *N) {
    int64_t n = 0;
    for (int j = 0; j < nprob; ++j) n += (int64_t)tiles128(N[j]) * BN;
    return rows * n * 4 <= kAccumBytes;
}
static int64_t stream_partial_bytes(const StreamPlan &sp) { return (int64_t)sp.slots * BN * sp.nb * 4; }

// Gated pair: one fp32 tile per tile of either weight, where the first finisher of a pair leaves its values.
static int64_t stream_gate_bytes(const StreamPlan &sp) { return (int64_t)sp.tiles_total * BN * sp.nb * 4; }

int64_t decode_workspace_bytes_multi(int64_t rows, int64_t K, int nprob, const int64_t *N, bool compact, bool gated = false, bool smem_operand = false) {
    const StreamPlan sp = stream_plan(rows, K, nprob, N, smem_operand);
    if (gated) return kCounterBytes + kAccumBytes + stream_partial_bytes(sp) + stream_gate_bytes(sp);
    if (!sp.shared_tiles) return 0;
    return kCounterBytes + (compact ? 0 : kAccumBytes) + stream_partial_bytes(sp);
}

int64_t decode_workspace_bytes_compact(int64_t rows, int64_t K, int64_t N) { return decode_workspace_bytes_multi(rows, K, 1, &N, true); }

int64_t decode_workspace_bytes(int64_t rows, int64_t K, int64_t N, bool smem_operand) { return decode_workspace_bytes_multi(rows, K, 1, &N, false, false, smem_operand); }

// Fills the launch arguments of one ttb_matmul_multi-shaped piece of work. `zero_bytes`: how much of the head of the
// workspace must be zero before the launch (the caller clears it unless it is known to be).
static int32_t prepare_decode_args(DecodeArgs &p, int &nb_out, int64_t &zero_bytes, const void *a, int nprob, const void *const *w, int w_dtype,
                                   const void *const *bias, void *const *out, int out_dtype, int64_t rows, int64_t K, const int64_t *N, int act,
                                   int flags, void *workspace, int64_t workspace_bytes, bool compact, const ttb_peer_gather *gather,
                                   const ttb_peer_wait_t *wait) {
    (void)w_dtype;
    p = DecodeArgs{};
    p.depends_on = -1;
    zero_bytes = 0;
    p.a = (const uint16_t *)a;
    p.K = K; p.Kt = (int)(K / 32); p.nkb = (int)(K / BK);
    p.act = act; p.out_dtype = out_dtype;
    p.a_row_major = (flags & TTB_MM_A_ROW_MAJOR) != 0;
    p.out_row_major = (flags & TTB_MM_OUT_ROW_MAJOR) != 0;
    if (int32_t rc = status_word_address(&p.status)) return rc;
    p.wait_limit = g_wait_limit_cycles;
    if (wait) {
        p.wait_arrived = wait->arrived; p.wait_expected = wait->expected;
    }
    const bool smem_operand = (flags & TTB_MM_DECODE_SMEM_OPERAND) != 0;
    const int nb = decode_rows_per_block(rows, smem_operand, any_ragged(nprob, N));
    // streamed decomposition
    const StreamPlan sp = stream_plan(rows, K, nprob, N, smem_operand);
    p.nprob = nprob;
    int t0 = 0;
    int64_t nsum = 0;
    for (int j = 0; j < nprob; ++j) {
        p.wv[j] = (const uint8_t *)w[j];
        p.biasv[j] = (const uint16_t *)(bias ? bias[j] : nullptr);
        p.outv[j] = out[j];
        p.Nv[j] = N[j];
        p.tstart[j] = t0;
        t0 += tiles128(N[j]);
        nsum += (int64_t)tiles128(N[j]) * BN;
    }
    p.tstart[nprob] = t0;
    p.sk_grid = sp.grid; p.sk_gran = sp.gran; p.sk_upt = sp.upt;
    p.sk_units = (int)sp.units; p.sk_q = (int)(sp.units / sp.grid); p.sk_r = (int)(sp.units % sp.grid);
    p.sk_waves = sp.waves; p.sk_rem_tile0 = sp.rem_tile0; p.sk_tiles = sp.tiles_total;
    p.splits = sp.pieces; p.kb_per_split = sp.kbps;
    p.ordered = compact || (flags & TTB_MM_DETERMINISTIC) != 0 || !stream_accumulate_ok(rows, nprob, N);
    const bool gated = (flags & TTB_MM_GATED) != 0;
    if (gated) {
        if (nprob != 2 || N[0] != N[1]) return fail(TTB_E_INVALID, "ttb_matmul_multi: a gated launch takes two weights of one shape");
        if (nb != 32 || compact || (flags & TTB_MM_DECODE_SMEM_OPERAND))
            return fail(TTB_E_UNSUPPORTED, "ttb_matmul_multi: the gated form serves row counts that are odd multiples of 32 (32, 96, 160, 224)");
        if (sp.tiles_total + sp.tiles_total / 2 > kSyncInt0) return fail(TTB_E_UNSUPPORTED, "ttb_matmul_multi: too many tiles for a gated launch");
        p.gated = 1;
    }
    if (gather) {
        if (N[0] % BN) return fail(TTB_E_UNSUPPORTED, "ttb_matmul: a gathered output needs a column count that is a multiple of 128");
        p.ranks = gather->ranks; p.rank = gather->rank;
        p.outv[0] = gather->out[gather->rank];
        p.out_n0 = (int64_t)gather->rank * N[0]; p.out_N = (int64_t)gather->ranks * N[0]; p.out_Nt = (int)(p.out_N / 32);
        for (int r = 0; r < gather->ranks; ++r) {
            p.peer_out[r] = (uint16_t *)gather->out[r];
            p.peer_arrived[r] = gather->arrived[r];
        }
        p.expected = gather->expected;
        p.launch_arrivals = (unsigned)(gather->ranks * (int)(N[0] / BN) * sp.rchunks);
    }
    if (sp.shared_tiles || gated) {
        const int64_t need = decode_workspace_bytes_multi(rows, K, nprob, N, compact, gated, smem_operand);
        if (!workspace || workspace_bytes < need)
            return fail(TTB_E_WORKSPACE, "ttb_matmul: this shape needs %lld bytes of workspace, got %lld", (long long)need,
                        (long long)workspace_bytes);
        if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return fail(TTB_E_INVALID, "ttb_matmul: workspace must be 256-byte aligned");
        p.counters = (int *)workspace;
        p.accum = (float *)((uint8_t *)workspace + kCounterBytes);
        p.partial = (float *)((uint8_t *)workspace + kCounterBytes + (compact ? 0 : kAccumBytes));
        if (gated) {
            p.gate = (float *)((uint8_t *)workspace + kCounterBytes + kAccumBytes + stream_partial_bytes(sp));
            p.gate_counters = p.counters + sp.tiles_total;
        }
        // counters always; in accumulate mode also the tiles this launch adds into
        zero_bytes = kCounterBytes + (p.ordered ? 0 : rows * nsum * 4);
    }
    nb_out = nb;
    return TTB_OK;
}

int32_t launch_matmul_decode_multi(const void *a, int nprob, const void *const *w, int w_dtype, const void *const *bias, void *const *out,
                                   int out_dtype, int64_t rows, int64_t K, const int64_t *N, int act, int flags, void *workspace,
                                   int64_t workspace_bytes, bool counters_are_zero, bool compact, cudaStream_t stream,
                                   const ttb_peer_gather *gather, const ttb_peer_wait_t *wait) {
    DecodeArgs p;
    int nb = 0;
    int64_t zero_bytes = 0;
    if (int32_t rc = prepare_decode_args(p, nb, zero_bytes, a, nprob, w, w_dtype, bias, out, out_dtype, rows, K, N, act, flags, workspace,
                                         workspace_bytes, compact, gather, wait))
        return rc;
    bool overlap = (flags & TTB_MM_WEIGHTS_RESIDENT) != 0;
    if (zero_bytes > 0 && !counters_are_zero) {
        TTB_CUDA_TRY(cudaMemsetAsync(workspace, 0, (size_t)zero_bytes, stream));
        overlap = false;   // only kernels may separate a launch from the one it overlaps with
    }
    // the weights reach the MMA through tensor memory (blocks of one or two tile rows), on request through shared memory
    for (int j = 0; j < nprob; ++j)
        if (N[j] % BN && (flags & TTB_MM_DECODE_SMEM_OPERAND))
            return fail(TTB_E_UNSUPPORTED, "ttb_matmul: the shared-memory-operand kernel needs column counts that are multiples of 128");
    if (!(flags & TTB_MM_DECODE_SMEM_OPERAND))
        return launch_decode_tmem(&p, 1, w_dtype, nb, p.counters ? p.counters + kSyncInt0 : nullptr, overlap, stream);
    return launch_decode_stream(p, w_dtype, nb, overlap, stream);
}

// Several ttb_matmul_multi-shaped stages in one launch of the tensor-memory kernel. The workspace is cut into one slice per
// stage (blocks can be in different stages at the same time); the first slice's counter region also carries the launch's
// own counters.
int64_t decode_sequence_workspace_bytes(int64_t rows, int count, const ttb_matmul_stage *st) {
    int64_t total = kCounterBytes;   // the launch's counters (and nothing else, so that a stage without scratch needs none)
    for (int s = 0; s < count; ++s) {
        const bool gated = (st[s].flags & TTB_MM_GATED) != 0;
        total += (decode_workspace_bytes_multi(rows, st[s].K, st[s].count, st[s].N, false, gated) + 255) & ~int64_t(255);
    }
    return total;
}

int32_t launch_matmul_decode_sequence(const ttb_matmul_stage *st, int count, int w_dtype, int64_t rows, int flags, void *workspace,
                                      int64_t workspace_bytes, cudaStream_t stream) {
    if (count < 1 || count > kMaxSequenceStages) return fail(TTB_E_INVALID, "ttb_matmul_sequence: 1..%d stages, got %d", kMaxSequenceStages, count);
    if (rows % 64 == 0)
        return fail(TTB_E_UNSUPPORTED, "ttb_matmul_sequence: serves row counts that are odd multiples of 32 (32, 96, 160, 224)");
    const int64_t need = decode_sequence_workspace_bytes(rows, count, st);
    if (!workspace || workspace_bytes < need)
        return fail(TTB_E_WORKSPACE, "ttb_matmul_sequence: needs %lld bytes of workspace, got %lld", (long long)need, (long long)workspace_bytes);
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return fail(TTB_E_INVALID, "ttb_matmul_sequence: workspace must be 256-byte aligned");
    // Blocks of a later stage wait for blocks of an earlier one: every block of the launch must get an SM of its own.
    int dev = 0, sms = 0;
    TTB_CUDA_TRY(cudaGetDevice(&dev));
    TTB_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    static DecodeArgs args[kMaxSequenceStages];
    const bool zeroed = (flags & TTB_MM_WORKSPACE_ZEROED) != 0;
    bool overlap = (flags & TTB_MM_WEIGHTS_RESIDENT) != 0;
    if (!zeroed) {
        TTB_CUDA_TRY(cudaMemsetAsync(workspace, 0, (size_t)kCounterBytes, stream));
        overlap = false;
    }
    uint8_t *ws = (uint8_t *)workspace + kCounterBytes;
    for (int s = 0; s < count; ++s) {
        const ttb_matmul_stage &g = st[s];
        const int sflags = g.flags & (TTB_MM_A_ROW_MAJOR | TTB_MM_OUT_ROW_MAJOR | TTB_MM_DETERMINISTIC | TTB_MM_GATED);
        const int64_t slice = (decode_workspace_bytes_multi(rows, g.K, g.count, g.N, false, (sflags & TTB_MM_GATED) != 0) + 255) & ~int64_t(255);
        int nb = 0;
        int64_t zero_bytes = 0;
        if (int32_t rc = prepare_decode_args(args[s], nb, zero_bytes, g.a, g.count, g.w, w_dtype, g.bias, g.out, g.out_dtype, rows, g.K, g.N,
                                             g.activation, sflags, slice ? ws : nullptr, slice, /*compact=*/false, g.gather, g.wait))
            return rc;
        if (args[s].sk_grid > sms)
            return fail(TTB_E_UNSUPPORTED, "ttb_matmul_sequence: the plan uses %d blocks, the device has %d multiprocessors", args[s].sk_grid, sms);
        if (g.input_from >= s || g.input_from < -1) return fail(TTB_E_INVALID, "ttb_matmul_sequence: stage %d: input_from must name an earlier stage or be -1", s);
        args[s].depends_on = g.input_from;
        if (g.input_from >= 0) args[g.input_from].count_done = 1;
        if (zero_bytes > 0 && !zeroed) TTB_CUDA_TRY(cudaMemsetAsync(ws, 0, (size_t)zero_bytes, stream));
        ws += slice;
    }
    return launch_decode_tmem(args, count, w_dtype, 32, (int *)workspace, overlap, stream);
}

int32_t launch_matmul_decode(const void *a, const void *w, int w_dtype, const void *bias, void *out, int out_dtype,
                             int64_t rows, int64_t K, int64_t N, int act, int flags, void *workspace,
                             int64_t workspace_bytes, bool counters_are_zero, bool compact, cudaStream_t stream,
                             const ttb_peer_gather *gather, const ttb_peer_wait_t *wait) {
    return launch_matmul_decode_multi(a, 1, &w, w_dtype, &bias, &out, out_dtype, rows, K, &N, act, flags, workspace, workspace_bytes,
                                      counters_are_zero, compact, stream, gather, wait);
}

int32_t read_and_clear_status(cudaStream_t stream) {
    TTB_CUDA_TRY(cudaStreamSynchronize(stream));
    int v = 0;
    TTB_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int)));
    if (v != 0) {
        int zero = 0;
        TTB_CUDA_TRY(cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int)));
        return fail(TTB_E_TIMEOUT, "a bounded device-side wait ran out (wait site %d)", v);
    }
    return TTB_OK;
}

}  // namespace ttb

// ---- decode matmul for callers that must not allocate ---------------------------------------------------------------
// Scratch for the split-K reduction lives in this library's own device image instead of a caller-provided buffer.
// Every GPU that loads the library holds these bytes until the process exits.
#define TTB_STATIC_SCRATCH_BYTES (65536 + (16 << 20))
static __device__ __align__(256) unsigned char g_static_scratch[TTB_STATIC_SCRATCH_BYTES];

extern "C" int64_t ttb_matmul_decode_static_scratch_bytes(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int64_t N) {
    using namespace ttb;
    if (batch <= 0 || M <= 0 || K <= 0 || N <= 0 || N % BN || !decode_supported(w_dtype, batch * M, K, N)) return -1;
    return decode_workspace_bytes_compact(batch * M, K, N);
}

extern "C" int32_t ttb_matmul_decode_static(const void *a, int32_t a_dtype, const void *w, int32_t w_dtype, const void *bias,
                                            void *out, int32_t out_dtype, int64_t batch, int64_t M, int64_t K, int64_t N,
                                            int32_t act, int32_t flags, void *stream) {
    using namespace ttb;
    if (!a || !w || !out) return fail(TTB_E_INVALID, "ttb_matmul_decode_static: null tensor pointer");
    if (a_dtype != TTB_BFLOAT16) return fail(TTB_E_UNSUPPORTED, "ttb_matmul_decode_static: activations must be bfloat16");
    if (out_dtype != TTB_BFLOAT16 && out_dtype != TTB_FLOAT32)
        return fail(TTB_E_UNSUPPORTED, "ttb_matmul_decode_static: output must be bfloat16 or float32");
    if (batch <= 0 || M <= 0 || K <= 0 || N <= 0 || M % 32 || K % 32 || N % 32)
        return fail(TTB_E_INVALID, "ttb_matmul_decode_static: batch, M, K, N must be positive and M, K, N multiples of 32");
    if (act < TTB_ACT_NONE || act > TTB_ACT_SILU) return fail(TTB_E_INVALID, "ttb_matmul_decode_static: unknown activation %d", act);
    if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(TTB_E_INVALID, "ttb_matmul_decode_static: tensors must be 16-byte aligned");
    const int64_t rows = batch * M;
    if (N % BN || !decode_supported(w_dtype, rows, K, N))
        return fail(TTB_E_UNSUPPORTED,
                    "ttb_matmul_decode_static: only the decode shapes are served without allocation (bfloat8_b / bfloat4_b weights, "
                    "at most 256 rows, N a multiple of 128); use ttb_matmul for [%lld x %lld x %lld]",
                    (long long)rows, (long long)K, (long long)N);
    const int64_t need = decode_workspace_bytes_compact(rows, K, N);
    if (need > (int64_t)TTB_STATIC_SCRATCH_BYTES)
        return fail(TTB_E_WORKSPACE,
                    "ttb_matmul_decode_static: this shape needs %lld bytes of scratch, the built-in scratch holds %lld; use ttb_matmul "
                    "with a caller-provided workspace",
                    (long long)need, (long long)TTB_STATIC_SCRATCH_BYTES);
    // Set-up, once per device, with that device current: the array's name is only a host-side handle here, the kernel
    // needs the device address the runtime maps it to.
    static void *scratch_addr[64] = {};
    int dev = 0;
    TTB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TTB_E_UNSUPPORTED, "ttb_matmul_decode_static: device index %d is out of range", dev);
    if (!scratch_addr[dev]) {
        void *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr)
            return fail(TTB_E_CUDA, "ttb_matmul_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        scratch_addr[dev] = ptr;
    }
    // The array keeps whatever the previous call left. Only the arrival counters at its head must start at zero
    // (launch_matmul_decode clears them on the stream); the partial sums are fully rewritten before they are read.
    return launch_matmul_decode(a, w, w_dtype, bias, out, out_dtype, rows, K, N, act, flags & (TTB_MM_A_ROW_MAJOR | TTB_MM_OUT_ROW_MAJOR),
                                need > 0 ? scratch_addr[dev] : nullptr, need, /*counters_are_zero=*/false, /*compact=*/true, (cudaStream_t)stream,
                                nullptr, nullptr);
}

// ---- matmul with the all-gather in its epilogue ------------------------------------------------------------------------
extern "C" int64_t ttb_matmul_peer_workspace_bytes(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int64_t N) {
    using namespace ttb;
    if (batch <= 0 || M <= 0 || K <= 0 || N <= 0 || !decode_supported(w_dtype, batch * M, K, N)) return 0;
    return decode_workspace_bytes(batch * M, K, N, false);
}

extern "C" int32_t ttb_matmul_peer(const void *a, int32_t a_dtype, const void *w, int32_t w_dtype, const void *bias, void *out,
                                   int32_t out_dtype, int64_t batch, int64_t M, int64_t K, int64_t N, int32_t act, int32_t flags,
                                   void *workspace, int64_t workspace_bytes, const ttb_peer_gather *gather,
                                   const ttb_peer_wait_t *wait, void *stream) {
    using namespace ttb;
    if (!a || !w || (!out && !gather)) return fail(TTB_E_INVALID, "ttb_matmul_peer: null tensor pointer");
    if (a_dtype != TTB_BFLOAT16) return fail(TTB_E_UNSUPPORTED, "ttb_matmul_peer: activations must be bfloat16");
    if (batch <= 0 || M <= 0 || K <= 0 || N <= 0 || M % 32 || K % 32 || N % 32)
        return fail(TTB_E_INVALID, "ttb_matmul_peer: batch, M, K, N must be positive and M, K, N multiples of 32");
    if (act < TTB_ACT_NONE || act > TTB_ACT_SILU) return fail(TTB_E_INVALID, "ttb_matmul_peer: unknown activation %d", act);
    const int64_t rows = batch * M;
    if (!decode_supported(w_dtype, rows, K, N))
        return fail(TTB_E_UNSUPPORTED,
                    "ttb_matmul_peer: decode shapes only (bfloat8_b / bfloat4_b weights, at most 256 rows, N a multiple of 128), got "
                    "[%lld x %lld x %lld]", (long long)rows, (long long)K, (long long)N);
    if (gather) {
        if (gather->ranks < 2 || gather->ranks > TTB_MAX_RANKS || gather->rank < 0 || gather->rank >= gather->ranks)
            return fail(TTB_E_INVALID, "ttb_matmul_peer: ranks must be 2..%d and rank inside it", TTB_MAX_RANKS);
        if (out_dtype != TTB_BFLOAT16 || (flags & TTB_MM_OUT_ROW_MAJOR))
            return fail(TTB_E_UNSUPPORTED, "ttb_matmul_peer: the gathered output is bfloat16 in tile layout");
        if (!gather->expected) return fail(TTB_E_INVALID, "ttb_matmul_peer: null expected-arrivals counter");
        for (int r = 0; r < gather->ranks; ++r)
            if (!gather->out[r] || !gather->arrived[r] || (reinterpret_cast<uintptr_t>(gather->out[r]) & 15))
                return fail(TTB_E_INVALID, "ttb_matmul_peer: null or misaligned peer pointer for rank %d", r);
    } else if (out_dtype != TTB_BFLOAT16 && out_dtype != TTB_FLOAT32) {
        return fail(TTB_E_UNSUPPORTED, "ttb_matmul_peer: output must be bfloat16 or float32");
    }
    if (wait && (!wait->arrived || !wait->expected))
        return fail(TTB_E_INVALID, "ttb_matmul_peer: incomplete wait description");
    return launch_matmul_decode(a, w, w_dtype, bias, out, out_dtype, rows, K, N, act,
                                flags & (TTB_MM_A_ROW_MAJOR | TTB_MM_OUT_ROW_MAJOR | TTB_MM_DETERMINISTIC | TTB_MM_WEIGHTS_RESIDENT | TTB_MM_DECODE_SMEM_OPERAND),
                                workspace, workspace_bytes, (flags & TTB_MM_WORKSPACE_ZEROED) != 0, /*compact=*/false,
                                (cudaStream_t)stream, gather, wait);
}

// The work decomposition a launch would use, for callers that want to know the launch geometry (and for tests, which
// re-walk it on the CPU and check that every K block of every tile is covered exactly once).
extern "C" int32_t ttb_matmul_decode_plan(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int32_t count, const int64_t *N,
                                          int32_t *out, int32_t out_len) {
    using namespace ttb;
    if (!N || !out || out_len < 10) return fail(TTB_E_INVALID, "ttb_matmul_decode_plan: needs N and room for 10 values");
    if (batch <= 0 || M <= 0 || !decode_supported_multi(w_dtype, batch * M, K, count, N))
        return fail(TTB_E_UNSUPPORTED, "ttb_matmul_decode_plan: not a decode shape");
    const StreamPlan sp = stream_plan(batch * M, K, count, N);
    const int32_t v[10] = {sp.nb, sp.tiles_total, sp.grid, sp.pieces, sp.kbps, sp.waves, sp.rem_tile0, (int32_t)sp.units, sp.upt, sp.slots};
    for (int i = 0; i < 10; ++i) out[i] = v[i];
    return TTB_OK;
}

// ---- several weights, one activation, one launch ------------------------------------------------------------------------
extern "C" int64_t ttb_matmul_multi_workspace_bytes(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int32_t count, const int64_t *N) {
    using namespace ttb;
    if (!N || batch <= 0 || M <= 0 || !decode_supported_multi(w_dtype, batch * M, K, count, N)) return 0;
    return decode_workspace_bytes_multi(batch * M, K, count, N, false);
}

extern "C" int64_t ttb_matmul_gated_workspace_bytes(int32_t w_dtype, int64_t batch, int64_t M, int64_t K, int64_t N) {
    using namespace ttb;
    const int64_t Ns[2] = {N, N};
    if (batch <= 0 || M <= 0 || !decode_supported_multi(w_dtype, batch * M, K, 2, Ns)) return 0;
    return decode_workspace_bytes_multi(batch * M, K, 2, Ns, false, true);
}

namespace ttb {
// Argument checks shared by ttb_matmul_multi and the stages of ttb_matmul_sequence.
static int32_t validate_multi(const char *who, const void *a, int32_t a_dtype, int32_t count, const void *const *w, int32_t w_dtype,
                              void *const *out, int32_t out_dtype, int64_t rows, int64_t K, const int64_t *N, int32_t act, int32_t flags,
                              const ttb_peer_gather *gather, const ttb_peer_wait_t *wait) {
    if (!a || !w || !out || !N) return fail(TTB_E_INVALID, "%s: null pointer", who);
    if (count < 1 || count > TTB_MAX_GROUP) return fail(TTB_E_INVALID, "%s: count must be 1..%d", who, TTB_MAX_GROUP);
    if (a_dtype != TTB_BFLOAT16) return fail(TTB_E_UNSUPPORTED, "%s: activations must be bfloat16", who);
    if (out_dtype != TTB_BFLOAT16 && out_dtype != TTB_FLOAT32) return fail(TTB_E_UNSUPPORTED, "%s: output must be bfloat16 or float32", who);
    if (rows <= 0 || K <= 0 || rows % 32 || K % 32) return fail(TTB_E_INVALID, "%s: batch, M, K must be positive and M, K multiples of 32", who);
    if (act < TTB_ACT_NONE || act > TTB_ACT_SILU) return fail(TTB_E_INVALID, "%s: unknown activation %d", who, act);
    for (int j = 0; j < count; ++j) {
        if (!w[j] || (!out[j] && !(gather && j == 0) && !((flags & TTB_MM_GATED) && j == 1)))
            return fail(TTB_E_INVALID, "%s: null tensor pointer for weight %d", who, j);
        if (N[j] <= 0 || N[j] % 32) return fail(TTB_E_INVALID, "%s: N[%d] must be a positive multiple of 32", who, j);
        if ((reinterpret_cast<uintptr_t>(w[j]) | reinterpret_cast<uintptr_t>(out[j])) & 15)
            return fail(TTB_E_INVALID, "%s: tensors must be 16-byte aligned", who);
    }
    if (!decode_supported_multi(w_dtype, rows, K, count, N))
        return fail(TTB_E_UNSUPPORTED, "%s: decode shapes only (bfloat8_b / bfloat4_b weights, at most 256 rows, every N a multiple of 128 - of 32 for row counts that are odd multiples of 32)", who);
    if (gather) {
        if (gather->ranks < 2 || gather->ranks > TTB_MAX_RANKS || gather->rank < 0 || gather->rank >= gather->ranks)
            return fail(TTB_E_INVALID, "%s: ranks must be 2..%d and rank inside it", who, TTB_MAX_RANKS);
        if (out_dtype != TTB_BFLOAT16 || (flags & TTB_MM_OUT_ROW_MAJOR)) return fail(TTB_E_UNSUPPORTED, "%s: the gathered output is bfloat16 in tile layout", who);
        if (!gather->expected) return fail(TTB_E_INVALID, "%s: null expected-arrivals counter", who);
        for (int r = 0; r < gather->ranks; ++r)
            if (!gather->out[r] || !gather->arrived[r] || (reinterpret_cast<uintptr_t>(gather->out[r]) & 15))
                return fail(TTB_E_INVALID, "%s: null or misaligned peer pointer for rank %d", who, r);
    }
    if (wait && (!wait->arrived || !wait->expected)) return fail(TTB_E_INVALID, "%s: incomplete wait description", who);
    return TTB_OK;
}
}  // namespace ttb

extern "C" int32_t ttb_matmul_multi(const void *a, int32_t a_dtype, int32_t count, const void *const *w, int32_t w_dtype,
                                    const void *const *bias, void *const *out, int32_t out_dtype, int64_t batch, int64_t M, int64_t K,
                                    const int64_t *N, int32_t act, int32_t flags, void *workspace, int64_t workspace_bytes,
                                    const ttb_peer_gather *gather, const ttb_peer_wait_t *wait, void *stream) {
    using namespace ttb;
    if (batch <= 0 || M <= 0 || M % 32) return fail(TTB_E_INVALID, "ttb_matmul_multi: batch, M, K must be positive and M, K multiples of 32");
    const int64_t rows = batch * M;
    if (int32_t rc = validate_multi("ttb_matmul_multi", a, a_dtype, count, w, w_dtype, out, out_dtype, rows, K, N, act, flags, gather, wait)) return rc;
    return launch_matmul_decode_multi(a, count, w, w_dtype, bias, out, out_dtype, rows, K, N, act,
                                      flags & (TTB_MM_A_ROW_MAJOR | TTB_MM_OUT_ROW_MAJOR | TTB_MM_DETERMINISTIC | TTB_MM_WEIGHTS_RESIDENT | TTB_MM_DECODE_SMEM_OPERAND | TTB_MM_GATED),
                                      workspace, workspace_bytes, (flags & TTB_MM_WORKSPACE_ZEROED) != 0, /*compact=*/false,
                                      (cudaStream_t)stream, gather, wait);
}

// ---- several such launches as the stages of one --------------------------------------------------------------------------
extern "C" int64_t ttb_matmul_sequence_workspace_bytes(int32_t w_dtype, int64_t batch, int64_t M, const ttb_matmul_stage *stages, int32_t count) {
    using namespace ttb;
    if (!stages || count < 1 || count > kMaxSequenceStages || batch <= 0 || M <= 0) return 0;
    for (int s = 0; s < count; ++s)
        if (!decode_supported_multi(w_dtype, batch * M, stages[s].K, stages[s].count, stages[s].N)) return 0;
    return decode_sequence_workspace_bytes(batch * M, count, stages);
}

extern "C" int32_t ttb_matmul_sequence(const ttb_matmul_stage *stages, int32_t count, int32_t a_dtype, int32_t w_dtype, int64_t batch, int64_t M,
                                       int32_t flags, void *workspace, int64_t workspace_bytes, void *stream) {
    using namespace ttb;
    if (!stages) return fail(TTB_E_INVALID, "ttb_matmul_sequence: null stage list");
    if (count < 1 || count > kMaxSequenceStages) return fail(TTB_E_INVALID, "ttb_matmul_sequence: 1..%d stages, got %d", kMaxSequenceStages, count);
    if (batch <= 0 || M <= 0 || M % 32) return fail(TTB_E_INVALID, "ttb_matmul_sequence: batch and M must be positive and M a multiple of 32");
    const int64_t rows = batch * M;
    for (int s = 0; s < count; ++s) {
        const ttb_matmul_stage &g = stages[s];
        if (int32_t rc = validate_multi("ttb_matmul_sequence", g.a, a_dtype, g.count, g.w, w_dtype, g.out, g.out_dtype, rows, g.K, g.N, g.activation,
                                        g.flags, g.gather, g.wait))
            return rc;
        if (g.input_from >= 0) {
            if (g.input_from >= s) return fail(TTB_E_INVALID, "ttb_matmul_sequence: stage %d: input_from must name an earlier stage", s);
            const ttb_matmul_stage &f = stages[g.input_from];
            if (f.out_dtype != TTB_BFLOAT16 || ((f.flags & TTB_MM_OUT_ROW_MAJOR) != 0) != ((g.flags & TTB_MM_A_ROW_MAJOR) != 0))
                return fail(TTB_E_INVALID, "ttb_matmul_sequence: stage %d reads stage %d's output, which must be bfloat16 in the layout stage %d expects", s,
                            g.input_from, s);
        }
    }
    return launch_matmul_decode_sequence(stages, count, w_dtype, rows, flags & (TTB_MM_WORKSPACE_ZEROED | TTB_MM_WEIGHTS_RESIDENT), workspace,
                                         workspace_bytes, (cudaStream_t)stream);
}

namespace {
__global__ void peer_wait_kernel(const uint32_t *arrived, const uint32_t *expected_ptr, int *status, long long limit) {
    const uint32_t expected = *reinterpret_cast<const volatile uint32_t *>(expected_ptr);
    const long long t0 = clock64();
    while ((int)(ttb::ld_acquire_sys(arrived) - expected) < 0) {
        if (clock64() - t0 > limit) {
            atomicCAS(status, 0, 7);
            return;
        }
        __nanosleep(100);
    }
}
}  // namespace

extern "C" int32_t ttb_set_wait_limit_cycles(int64_t cycles) {
    if (cycles < 0) return ttb::fail(TTB_E_INVALID, "ttb_set_wait_limit_cycles: the limit must be zero (defaults) or positive");
    ttb::g_wait_limit_cycles = cycles;
    return TTB_OK;
}

extern "C" int32_t ttb_peer_wait(const ttb_peer_wait_t *wait, void *stream) {
    using namespace ttb;
    if (!wait || !wait->arrived || !wait->expected) return fail(TTB_E_INVALID, "ttb_peer_wait: incomplete wait description");
    int *status = nullptr;
    if (int32_t rc = status_word_address(&status)) return rc;
    const long long limit = wait_limit_cycles() > 0 ? wait_limit_cycles() : 20000000000LL;
    peer_wait_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(wait->arrived, wait->expected, status, limit);
    TTB_LAUNCH_CHECK("peer_wait");
    return TTB_OK;
}
