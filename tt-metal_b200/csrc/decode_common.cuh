// Pieces shared by the two decode (small row count) matmul kernels: launch arguments, activation addressing and
// the epilogue's finish-and-store step.
#pragma once
#include <cuda.h>

#include "epilogue.cuh"
#include "sm100_ptx.cuh"

namespace ttb {

struct DecodeArgs;
constexpr int kMaxSequenceStages = 4;   // stages (ttb_matmul_multi calls) one launch can hold
// One tiled tensor map per weight of a launch: the packed weight seen as [K blocks][tiles per row][tile as 8-byte words], so
// that a producer thread fetches the stages of a group (`group` K blocks x four tiles) with ONE copy instruction.
struct alignas(64) WeightMaps {
    CUtensorMap m[TTB_MAX_GROUP];
};
int32_t make_weight_maps(const DecodeArgs &p, int fmt, WeightMaps &maps, int group = 3);
// The activation [rows, K] (tiled or row-major bf16) as a tensor map whose box is three K blocks of 32 rows, delivered in
// the MMA's K-major operand layout (`group` K blocks of 32 rows) with the 32-byte swizzle: [K block][16-column half][row][16 values].
struct alignas(64) ActMap {
    CUtensorMap m;
};
int32_t make_act_map(const DecodeArgs &p, int64_t rows, ActMap &map, int group = 3);

struct DecodeArgs {
    const uint8_t *w;
    const uint16_t *a;
    const uint16_t *bias;
    void *out;
    float *partial;   // ordered mode: one fp32 partial per split; accumulate mode: unused
    float *accum;     // accumulate mode: one fp32 tile per output tile, zero between launches
    int *counters;
    int64_t K, N;
    int Kt, Nt;
    int nkb, kb_per_split, splits;
    int act, out_dtype, a_row_major, out_row_major;
    int ordered;      // 1: add the split-K partials in split order (bit-reproducible); 0: red.add into `accum`
    int *status;  // device status word raised by bounded waits that run out
    // ---- output placement: the result is columns [out_n0, out_n0 + N) of a tensor with out_Nt tiles (or out_N columns
    // in row-major) per row; a plain matmul has out_n0 = 0, out_Nt = Nt, out_N = N ----
    int64_t out_n0, out_N;
    int out_Nt;
    // ---- gather epilogue (ranks > 1): every finished tile is also stored into the same columns of the other ranks'
    // copies of the output, then counted on every rank's arrival counter ----
    int ranks, rank;
    uint16_t *peer_out[TTB_MAX_RANKS];
    unsigned *peer_arrived[TTB_MAX_RANKS];
    unsigned *expected;        // this rank's running total of arrivals its gather point will have seen after this launch
    unsigned launch_arrivals;  // ranks x output tiles per rank
    // ---- wait before the first activation load: *wait_arrived must reach *wait_expected ----
    const unsigned *wait_arrived;
    const unsigned *wait_expected;
    // ---- streamed decomposition (matmul_decode_stream.cu): up to four weights share the activation; their 128-column
    // tiles form one list (per row chunk). sk_grid persistent blocks first take whole tiles, round by round, then share
    // the remaining tiles, whose K-blocks are cut into units of sk_gran K-blocks and dealt out evenly, in order ----
    int nprob;
    const uint8_t *wv[TTB_MAX_GROUP];
    const uint16_t *biasv[TTB_MAX_GROUP];
    void *outv[TTB_MAX_GROUP];
    int64_t Nv[TTB_MAX_GROUP];
    int tstart[TTB_MAX_GROUP + 1];   // first 128-column tile of each weight in the list; tstart[nprob] = tiles per row chunk
    int sk_grid, sk_gran, sk_upt;    // blocks, K-blocks per unit, units per tile
    int sk_waves, sk_rem_tile0;      // rounds of whole tiles (tile = round * sk_grid + block), first tile of the split remainder
    int sk_tiles;                    // tiles in the list (all row chunks)
    int sk_units, sk_q, sk_r;        // units of the streamed remainder; units / blocks and units % blocks
    // ---- gated pair (two weights, out = act(a w0 + b0) * (a w1 + b1)): whoever finishes a tile of either weight leaves its
    // fp32 values in `gate` and takes a ticket on the pair's counter; the second one forms the product and stores it ----
    int gated;
    float *gate;
    int *gate_counters;
    // ---- stages of one launch (matmul_decode_tmem.cu): the earlier stage whose output is this stage's activation (-1: none),
    // and whether this stage counts its stored tiles for a later one ----
    int depends_on, count_done;
    // ---- limit of the bounded waits in SM clocks (0 = the built-in defaults), set by ttb_set_wait_limit_cycles ----
    long long wait_limit;
};

// Limits of the two kinds of bounded waits of a launch. The barrier waits inside a block outlast the wait for the peers:
// the roles downstream of the expand warps sit in barrier waits while those wait for activations from other GPUs.
__device__ __forceinline__ long long peer_wait_limit(const DecodeArgs &p) { return p.wait_limit > 0 ? p.wait_limit : 20000000000LL; }
__device__ __forceinline__ long long barrier_wait_limit(const DecodeArgs &p) {
    if (p.wait_limit > 0) return 2 * p.wait_limit + 1000000LL;
    return p.wait_arrived ? 25000000000LL : 2000000000LL;
}

// Where a finished tile goes: one weight's output tensor (or its slice of a gathered tensor).
struct OutView {
    void *out;
    const uint16_t *bias;
    int64_t n0, N;   // first column of the slice inside the output tensor, and the output tensor's columns
    int Nt;          // 32-column tiles per row of the output tensor
};
__device__ __forceinline__ OutView out_view_of(const DecodeArgs &p) { return OutView{p.out, p.bias, p.out_n0, p.out_N, p.out_Nt}; }

// System-scope release / acquire on counters that other GPUs write or read over NVLink.
__device__ __forceinline__ void red_relaxed_sys_add(unsigned *addr, unsigned v) {
    asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *addr) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    return v;
}

// Bounded wait for the peers' slices of a gathered activation (one lane calls it). Returns false and raises the
// status word after `limit_cycles`, or as soon as another thread of the block gave up.
__device__ __forceinline__ bool peer_wait(const DecodeArgs &p, volatile int *abort_flag, int code) {
    if (!p.wait_arrived) return true;
    const long long limit_cycles = peer_wait_limit(p);
    const unsigned expected = *reinterpret_cast<const volatile unsigned *>(p.wait_expected);
    const long long t0 = clock64();
    for (unsigned spin = 1;; ++spin) {
        if ((int)(ld_acquire_sys(p.wait_arrived) - expected) >= 0) return true;
        if ((spin & 15u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit_cycles) {
                *abort_flag = 1;
                atomicCAS(p.status, 0, code);
                return false;
            }
        }
        __nanosleep(64);
    }
}

// The same against a total the caller computed (stages of one launch: what the gather point had been told to expect before
// the launch plus the shares of the launch's own earlier stages).
__device__ __forceinline__ bool peer_wait_for(const DecodeArgs &p, unsigned expected, volatile int *abort_flag, int code) {
    const long long limit_cycles = peer_wait_limit(p);
    const long long t0 = clock64();
    for (unsigned spin = 1;; ++spin) {
        if ((int)(ld_acquire_sys(p.wait_arrived) - expected) >= 0) return true;
        if ((spin & 15u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit_cycles) {
                *abort_flag = 1;
                atomicCAS(p.status, 0, code);
                return false;
            }
        }
        __nanosleep(64);
    }
}
// Bounded wait until a counter of this GPU (tiles an earlier stage of the launch has stored) reaches `target`.
__device__ __forceinline__ bool count_wait(const int *counter, int target, const DecodeArgs &p, volatile int *abort_flag, int code) {
    const long long limit_cycles = peer_wait_limit(p);
    const long long t0 = clock64();
    for (unsigned spin = 1;; ++spin) {
        int v;
        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if (v >= target) return true;
        if ((spin & 15u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit_cycles) {
                *abort_flag = 1;
                atomicCAS(p.status, 0, code);
                return false;
            }
        }
        __nanosleep(64);
    }
}

// Adds four floats to global memory with one vector reduction (no return value, any order).
__device__ __forceinline__ void red_add_f32x4(float *addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Global element offset of the 8-element activation chunk (row r, columns k..k+7).
__device__ __forceinline__ int64_t act_chunk_offset(const DecodeArgs &p, int64_t r, int64_t k) {
    if (p.a_row_major) return r * p.K + k;
    return ((r >> 5) * p.Kt + (k >> 5)) * 1024 + 256 * (2 * (int)((r & 31) >> 4) + (int)((k & 31) >> 4)) + 16 * (int)(r & 15) +
           (int)(k & 15);
}

// Bias, activation and store of 16 consecutive rows (row0 + col0 .. + 15, col0 a multiple of 16) of output column n.
// In the tiled layout those 16 elements sit 16 apart inside one face, in the row-major layout N apart.
// Element offset of the chunk (row r, K-block 0, 8-element chunk kc of the block's 32 columns) and the constant step from
// one K-block to the next: a K-block is one tile column in the tiled layout (1024 elements on), 32 elements in row-major.
__device__ __forceinline__ int64_t act_chunk_base(const DecodeArgs &p, int64_t r, int kc) {
    if (p.a_row_major) return r * p.K + kc * 8;
    return (r >> 5) * p.Kt * 1024 + 256 * (2 * (int)((r & 31) >> 4) + (kc >> 1)) + 16 * (int)(r & 15) + (kc & 1) * 8;
}
__device__ __forceinline__ int act_chunk_step(const DecodeArgs &p) { return p.a_row_major ? 32 : 1024; }

// `stage` (gather epilogue only, bf16 tiled output) receives a copy at the element's position inside the block's own
// [rows of the block, 128 columns] tiled slab, from where whole tiles are sent to the other ranks.
template <int ACT>
__device__ __forceinline__ void finish_and_store_t(const DecodeArgs &p, const OutView &ov, const float (&v)[16], int64_t row0, int col0,
                                                   int64_t n, uint16_t *stage) {
    const float bias = ov.bias ? bias_at(ov.bias, n) : 0.0f;
    const int64_t r0 = row0 + col0;
    const int64_t base = p.out_row_major ? r0 * ov.N + ov.n0 + n : tiled_offset(r0, ov.n0 + n, ov.Nt);
    const int64_t stride = p.out_row_major ? ov.N : 16;
    if (p.out_dtype == TTB_FLOAT32) {
        float *o = reinterpret_cast<float *>(ov.out) + base;
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j * stride] = apply_activation_t<ACT>(v[j] + bias);
    } else {
        uint16_t *o = reinterpret_cast<uint16_t *>(ov.out) + base;
        if (stage) {
            const int c = (int)(n & 127);
            uint16_t *s = stage + ((col0 >> 5) * 4 + (c >> 5)) * 1024 + 256 * (2 * ((col0 & 31) >> 4) + ((c & 31) >> 4)) + (c & 15);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const uint16_t b = f32_to_bf16_bits(apply_activation_t<ACT>(v[j] + bias));
                o[j * stride] = b;
                s[j * 16] = b;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j * stride] = f32_to_bf16_bits(apply_activation_t<ACT>(v[j] + bias));
        }
    }
}

template <int NB>
__device__ __forceinline__ void finish_and_store(const DecodeArgs &p, const OutView &ov, const float (&v)[16], int64_t row0, int col0,
                                                 int64_t n, uint16_t *stage = nullptr) {
    TTB_DISPATCH_ACT(p.act, finish_and_store_t<ACT>(p, ov, v, row0, col0, n, stage));
}
// The same as one out-of-line copy: a kernel that finishes tiles in several places would otherwise carry the activation x
// output-type x staging variants of the store loop at each of them, and its instruction footprint decides how long a
// short launch takes (instruction-fetch stalls dominated the profile of the inlined form).
template <int NB>
__device__ __noinline__ void finish_and_store_shared(const DecodeArgs &p, const OutView &ov, const float (&v)[16], int64_t row0, int col0,
                                                     int64_t n, uint16_t *stage) {
    TTB_DISPATCH_ACT(p.act, finish_and_store_t<ACT>(p, ov, v, row0, col0, n, stage));
}
template <int NB>
__device__ __forceinline__ void finish_and_store(const DecodeArgs &p, const float (&v)[16], int64_t row0, int col0, int64_t n,
                                                 uint16_t *stage = nullptr) {
    finish_and_store<NB>(p, out_view_of(p), v, row0, col0, n, stage);
}

// Gather epilogue, called by all `nthreads` epilogue threads of a block after the block has stored its finished
// [NB x 128] slab locally and into `stage`: sends the slab to every other rank with 16-byte stores (each 32-row tile row
// of the slab is 8 KiB contiguous in the tiled output) and counts the tile on every rank's arrival counter.
// Cost of the pieces, measured between two B200s over NVLink: a system-scope fence is ~1.7 us with nothing outstanding and
// ~3.6 us behind remote stores, a release-flavoured remote reduction costs as much as a fence, a relaxed one ~40 ns, and
// a flag needs ~1.25 us to be seen by the peer. Hence exactly one fence per tile: all threads store, a barrier orders
// them before thread 0, whose single fence (cumulative) precedes relaxed reductions on the counters.
template <int NB>
__device__ __forceinline__ void gather_send(const DecodeArgs &p, const uint16_t *stage, int64_t row0, int ntile, int tid, int nthreads) {
    // (the gathered tensor is the output of the first weight of the launch: p.out_n0 / p.out_Nt describe it)
    asm volatile("bar.sync 2, %0;" ::"r"(nthreads) : "memory");   // the slab is complete in shared memory
    constexpr int kVecPerRow = 4 * 1024 * 2 / 16;                  // 512 16-byte vectors per tile row of the slab
    const uint4 *src = reinterpret_cast<const uint4 *>(stage);
    for (int step = 1; step < p.ranks; ++step) {
        const int r = (p.rank + step) % p.ranks;
        for (int rt = 0; rt < NB / 32; ++rt) {
            uint4 *dst = reinterpret_cast<uint4 *>(p.peer_out[r] + (((row0 >> 5) + rt) * p.out_Nt + ((p.out_n0 >> 5) + ntile * 4)) * 1024);
            for (int i = tid; i < kVecPerRow; i += nthreads) dst[i] = src[rt * kVecPerRow + i];
        }
    }
    asm volatile("bar.sync 2, %0;" ::"r"(nthreads) : "memory");
    if (tid == 0) {
        __threadfence_system();
        for (int step = 1; step <= p.ranks; ++step) red_relaxed_sys_add(p.peer_arrived[(p.rank + step) % p.ranks], 1u);
    }
}

}  // namespace ttb
