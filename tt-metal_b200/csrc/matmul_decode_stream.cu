// Streamed weight matmul for small row counts (decode), persistent form:
//   out_j[rows, N_j] = act(a[rows, K] x W_j[K, N_j] + bias_j)   for up to four weights W_j that share the activation.
//
// Giving every block one 128-column tile and a fixed share of K leaves a quarter of the machine idle whenever the tile
// count does not fill the SMs in whole waves (112 tiles on 148 SMs), and makes every small projection of a decoder layer
// pay its own launch. Here the work is one list: the 128-column tiles of all weights of the launch. At most one persistent
// block per SM works through a few segments - (tile, K range) pairs, chosen by the host's plan (SegIter below) - with one
// uninterrupted stream of packed weight tiles: the producer thread keeps prefetching across segment borders, so only the
// first segment of a block pays the HBM latency. A tile whose K range is shared by several blocks is summed in fp32 from
// per-block partials in block order (few sharers, or deterministic mode) or with vector reductions (many sharers); the
// last block to arrive finishes it (bias, activation, store, optional store into the other ranks' copies).
//
// Roles (12 warps): warp 0 lane 0 streams packed tiles; warps 4 and 8 (lane 0) issue the MMAs of the first and second K
// step of every stage into their own accumulators; the nine warps with warp % 4 != 0 expand packed codes to bf16
// operands. Warps 4..11 also run the epilogue of every segment (TMEM lane quadrant = warp % 4): the MMA issuers take
// part, so no MMA can overwrite an accumulator that is still being read, while warps 1..3 keep expanding ahead and the
// producer keeps streaming. Every wait is bounded.
#include "decode_smem.cuh"

namespace ttb {

namespace {

using namespace ptx;
using namespace decode_smem;

constexpr int kEpiWarp0 = 4;                       // warps 4..11 run epilogues
constexpr int kEpiThreads = 256;

// Shared memory: the packed ring, the operand rings and a staging slab for the gather epilogue. With 128 rows per block the
// packed ring is shortened to make room.
template <int FMT, int NB>
struct StreamLayout {
    static constexpr int kPkG = NB == 128 ? 3 : kPkGroups;
    static constexpr int kPkSt = kGroup * kPkG;
    static constexpr int kBStageBytes = NB * BK * 2;
    static constexpr int kAbGroups = Ab<NB>::kGroups;
    static constexpr int kAbStages = Ab<NB>::kStages;
    static constexpr int pk = 0;
    static constexpr int a = pk + kPkSt * Pk<FMT>::kStageBytes;
    static constexpr int b = a + kAbStages * kAStageBytes;
    static constexpr int stage = b + kAbStages * kBStageBytes;   // [NB x 128] bf16, tiled
    static constexpr int bars = stage + NB * BN * 2;
    static constexpr int nbars = 2 * kPkG + 2 * kAbGroups + 1;
    static constexpr int misc = bars + 8 * nbars;                // tmem base, abort flag, last-block flag
    static constexpr int total = misc + 16;
    // Three teams of expand warps wait on the ring barriers with different phase parities; that is only right while a
    // waiter is at most one phase behind, i.e. while no ring has fewer groups than there are teams.
    static_assert(kExpandWarps / kGroup <= kPkG && kExpandWarps / kGroup <= kAbGroups, "ring shorter than the number of teams");
};

struct Seg {
    int tile;            // index into the tile list: row chunk * tiles per chunk + tile within the chunk
    int kb0;             // first K-block
    int nit;             // K-blocks
    int contributors;    // blocks (or pieces) that share the tile; 1 = this segment is the whole tile
    int slot0, slot;     // partial-sum slots of the tile's first contributor and of this segment
};

// The streamed remainder holds sk_units units; block b takes [b * q + min(b, r), ...) with q = units / grid, r = units % grid
// (the first r blocks take one unit more). All of it in 32-bit arithmetic: these run on single threads' critical paths.
__device__ __forceinline__ int unit_begin(const DecodeArgs &p, int b) { return b * p.sk_q + min(b, p.sk_r); }
__device__ __forceinline__ int block_of_unit(const DecodeArgs &p, int u) {
    const int big = p.sk_r * (p.sk_q + 1);
    return u < big ? u / (p.sk_q + 1) : p.sk_r + (u - big) / p.sk_q;
}

// A block's work, in order. Two decompositions:
//  * pieces (p.splits > 1): every tile is cut along K into p.splits equal pieces; piece q = part (q / tiles) of tile
//    (q % tiles); the blocks take pieces round by round (q = round * grid + block). Neighbouring blocks read the same K
//    rows of neighbouring tiles at the same time, which DRAM likes, and every block has one segment per round.
//  * whole tiles + streamed remainder (p.splits == 1): `sk_waves` rounds of whole tiles (tile = round * grid + block), then
//    the block's share of the remainder - the tiles from sk_rem_tile0 on, cut into units of sk_gran K-blocks and dealt
//    out evenly, in order, so that all blocks finish together.
struct SegIter {
    int w;
    int u, u_end;
    __device__ __forceinline__ void start(const DecodeArgs &p, int block) {
        w = 0;
        u = unit_begin(p, block);
        u_end = unit_begin(p, block + 1);
    }
    __device__ __forceinline__ bool next(const DecodeArgs &p, int block, Seg &s) {
        while (w < p.sk_waves) {
            const int q = w * p.sk_grid + block;
            ++w;
            if (q < p.sk_rem_tile0) {   // (in the pieces decomposition sk_rem_tile0 is the number of pieces)
                if (p.splits > 1) {
                    const int part = q / p.sk_tiles;
                    s.tile = q - part * p.sk_tiles;
                    s.kb0 = part * p.kb_per_split;
                    s.nit = min(p.nkb, s.kb0 + p.kb_per_split) - s.kb0;
                    s.contributors = p.splits;
                    s.slot0 = s.tile * p.splits;
                    s.slot = s.slot0 + part;
                } else {
                    s.tile = q; s.kb0 = 0; s.nit = p.nkb;
                    s.contributors = 1; s.slot0 = 0; s.slot = 0;
                }
                return true;
            }
        }
        if (u >= u_end) return false;
        const int rt = u / p.sk_upt;
        const int t0 = rt * p.sk_upt;
        const int e = min(u_end, t0 + p.sk_upt);
        s.tile = p.sk_rem_tile0 + rt;
        s.kb0 = (u - t0) * p.sk_gran;
        s.nit = min(p.nkb, (e - t0) * p.sk_gran) - s.kb0;
        const int fb = block_of_unit(p, t0);
        s.contributors = block_of_unit(p, t0 + p.sk_upt - 1) - fb + 1;
        s.slot0 = rt + fb;
        s.slot = rt + block;
        u = e;
        return true;
    }
};

// Which weight a tile of the list belongs to, its 128-column index inside that weight, and its row chunk.
struct TileRef {
    int prob, nt, rchunk;
};
__device__ __forceinline__ TileRef tile_ref(const DecodeArgs &p, int tile) {
    TileRef r;
    const int per = p.tstart[p.nprob];
    r.rchunk = tile / per;
    const int t = tile - r.rchunk * per;
    r.prob = 0;
#pragma unroll
    for (int j = 1; j < TTB_MAX_GROUP; ++j)
        if (j < p.nprob && t >= p.tstart[j]) r.prob = j;
    r.nt = t - p.tstart[r.prob];
    return r;
}

// What the epilogue of a segment needs from the kernel around it.
struct EpiCtx {
    uint8_t *smem;
    uint32_t tmem_base, accum_bar;
    volatile int *abort_flag;
    volatile int *last_flag;
    long long lim;
};

// Tiles shared by at most this many blocks are summed from per-block partials (plain stores, fixed order); tiles shared
// by more use fp32 reductions in L2 (when every block of a launch flushes a partial tile at once, 16 KiB of reductions
// per block cost several microseconds, plain stores a fraction of that).
constexpr int kPartialsUpTo = 4;

// ---------------- epilogue of one segment, run by warps 4..11 together; returns false after a wait that ran out ----------------
template <int FMT, int NB>
__device__ __forceinline__ bool stream_epilogue(const DecodeArgs &p, const EpiCtx c, const Seg s, const int seg_idx, bool ok) {
    using L = StreamLayout<FMT, NB>;
    constexpr int kAcc = BK / 16;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tid = threadIdx.x - 32 * kEpiWarp0;
    const int quad = warp & 3, half = (warp - kEpiWarp0) >> 2;
    constexpr int kColsPerWarp = NB / 2;
    int good = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0);
    if (lane == 0 && good) good = mbar_wait(c.accum_bar, (uint32_t)(seg_idx & 1), c.abort_flag, p.status, 5, c.lim) ? 1 : 0;
    const bool eok = __shfl_sync(0xffffffffu, good, 0) != 0;
    tc_fence_after_sync();
    const TileRef tr = tile_ref(p, s.tile);
    const int64_t row0 = (int64_t)tr.rchunk * NB;
    const int64_t n = (int64_t)tr.nt * BN + quad * 32 + lane;
    const bool gathered = p.ranks > 1 && tr.prob == 0;
    OutView ov;
    ov.out = p.outv[tr.prob];
    ov.bias = p.biasv[tr.prob];
    ov.n0 = gathered ? p.out_n0 : 0;
    ov.N = gathered ? p.out_N : p.Nv[tr.prob];
    ov.Nt = (int)(ov.N >> 5);
    uint16_t *const stage = gathered ? reinterpret_cast<uint16_t *>(c.smem + L::stage) : nullptr;
    const int contributors = s.contributors;
    const bool partials = p.ordered || contributors <= kPartialsUpTo;
    float *const acc_tile = p.accum + (int64_t)s.tile * BN * NB;
    // sum of the two accumulators, 16 consecutive columns of this lane's row
    auto read_accumulators = [&](int col0, float (&v)[16]) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.0f;
#pragma unroll
        for (int ac = 0; ac < kAcc; ++ac) {
            uint32_t r[16];
            tmem_ld16(c.tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ac * NB + col0), r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += __uint_as_float(r[j]);
        }
    };
    bool finished = contributors == 1;
    if (contributors > 1) {
        // phase 1: hand this block's share over (partial tile or reductions), then learn whether it arrived last
        if (eok) {
#pragma unroll
            for (int cc = 0; cc < kColsPerWarp / 16; ++cc) {
                const int col0 = half * kColsPerWarp + cc * 16;
                float v[16];
                read_accumulators(col0, v);
                if (partials) {
                    float4 *dst = reinterpret_cast<float4 *>(p.partial + ((int64_t)s.slot * BN + quad * 32 + lane) * NB + col0);
#pragma unroll
                    for (int j = 0; j < 4; ++j) __stcg(dst + j, make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
                } else {
                    float *dst = acc_tile + (quad * 32 + lane) * NB + col0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) red_add_f32x4(dst + 4 * j, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
        }
        // From this barrier on the accumulators are free: the MMA issuers are among its threads.
        tc_fence_before_sync();
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (tid == 0) {
            *c.last_flag = (atomicAdd(p.counters + s.tile, 1) == contributors - 1) ? 1 : 0;
            __threadfence();   // acquire side: what the other blocks published before their tickets is visible to every
                               // thread that passes the next barrier
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        finished = *c.last_flag != 0;
    }
    // phase 2: whoever holds the complete sum - the only block of an unshared tile, or the last arriver - finishes the tile
    if (finished && (eok || contributors > 1)) {
#pragma unroll
        for (int cc = 0; cc < kColsPerWarp / 16; ++cc) {
            const int col0 = half * kColsPerWarp + cc * 16;
            float v[16];
            if (contributors == 1) {
                read_accumulators(col0, v);
            } else if (partials) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                // Up to four blocks' partials per round: all loads of a round are issued before the first add (under the
                // weight stream a trip to L2 takes ~1.5 us, so rounds are what this costs); the adds stay in block order.
#pragma unroll 1
                for (int c0 = 0; c0 < contributors; c0 += 4) {
                    const float4 *src = reinterpret_cast<const float4 *>(
                        p.partial + ((int64_t)(s.slot0 + c0) * BN + quad * 32 + lane) * NB + col0);
                    constexpr int64_t kSlot = (int64_t)BN * NB / 4;   // float4 per slot
                    const int cnt = min(4, contributors - c0);
                    float4 x0[4], x1[4], x2[4], x3[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        x0[j] = __ldcg(src + j);
                        x1[j] = cnt > 1 ? __ldcg(src + kSlot + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                        x2[j] = cnt > 2 ? __ldcg(src + 2 * kSlot + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                        x3[j] = cnt > 3 ? __ldcg(src + 3 * kSlot + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    auto add = [&](const float4 (&x)[4]) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            v[4 * j] += x[j].x; v[4 * j + 1] += x[j].y; v[4 * j + 2] += x[j].z; v[4 * j + 3] += x[j].w;
                        }
                    };
                    add(x0);
                    if (cnt > 1) add(x1);
                    if (cnt > 2) add(x2);
                    if (cnt > 3) add(x3);
                }
            } else {
                float4 *acc = reinterpret_cast<float4 *>(acc_tile + (quad * 32 + lane) * NB + col0);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 x = __ldcg(acc + j);
                    v[4 * j] = x.x; v[4 * j + 1] = x.y; v[4 * j + 2] = x.z; v[4 * j + 3] = x.w;
                    acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);   // leave zeros for the next launch
                }
            }
            finish_and_store<NB>(p, ov, v, row0, col0, n, stage);
        }
        if (contributors > 1 && tid == 0) p.counters[s.tile] = 0;
    }
    if (contributors == 1) {
        // the accumulators are free from here on: the MMA issuers are among the threads of this barrier
        tc_fence_before_sync();
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
    }
    if (gathered) {
        // one decision for the whole group of threads, so that all of them take part in gather_send's barriers
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (tid == 0) *c.last_flag = (finished && *c.abort_flag == 0) ? 1 : 0;
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (*c.last_flag) gather_send<NB>(p, stage, row0, tr.nt, tid, kEpiThreads);   // ends with a barrier: the slab is free again
    }
    return eok;
}

template <int FMT, int NB>
__global__ void __launch_bounds__(kThreadsDecode, 1) matmul_decode_stream_kernel(const __grid_constant__ DecodeArgs p, const __grid_constant__ WeightMaps maps) {
    using L = StreamLayout<FMT, NB>;
    constexpr int TB = Pk<FMT>::kTileBytes;
    constexpr int kAcc = BK / 16;
    constexpr int kTmemCols = NB * kAcc < 32 ? 32 : NB * kAcc;
    constexpr int kAbGroups = L::kAbGroups;
    constexpr int kPkG = L::kPkG;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + L::bars;
    auto full_pk = [&](int s) { return bar0 + 8u * s; };
    auto empty_pk = [&](int s) { return bar0 + 8u * (kPkG + s); };
    auto full_ab = [&](int s) { return bar0 + 8u * (2 * kPkG + s); };
    auto empty_ab = [&](int s) { return bar0 + 8u * (2 * kPkG + kAbGroups + s); };
    const uint32_t accum_bar = bar0 + 8u * (2 * kPkG + 2 * kAbGroups);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::misc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::misc + 4);
    volatile int *last_flag = reinterpret_cast<volatile int *>(smem + L::misc + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int block = (int)blockIdx.x;
    // Limit of every barrier wait, in clocks: about a second, but longer than the peer wait when the activations come from
    // other GPUs (the roles downstream of the expand warps sit in barrier waits while those wait for the peers).
    const long long lim = barrier_wait_limit(p);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPkG; ++s) {
            mbar_init(full_pk(s), 1);
            mbar_init(empty_pk(s), kGroup);
        }
        for (int s = 0; s < kAbGroups; ++s) {
            mbar_init(full_ab(s), kGroup);
            mbar_init(empty_ab(s), 2);
        }
        mbar_init(accum_bar, 2);
        *abort_flag = 0;
        *last_flag = 0;
        fence_mbar_init();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(sbase + L::misc, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;
    // The next kernel on the stream may start streaming its weights while this grid drains; before grid_dep_wait() this
    // kernel reads nothing but packed weights.
    grid_dep_launch();
    const EpiCtx ectx = {smem, tmem_base, accum_bar, abort_flag, last_flag, lim};

    // Stages travel in groups of up to three (one barrier per group). A group never spans two segments: the last group of
    // a segment is simply shorter. The expand warp whose stage a short group lacks still takes its turn - it waits for the
    // group like the others and arrives on both barriers without expanding anything - so every barrier sees the same
    // arrivals in the same order for every group.
    if (warp == kProducerWarp) {
        // ---------------- producer: packed weight tiles -> shared-memory ring, across segment borders ----------------
        // One tensor-map copy per group. The whole warp walks the work list (addresses stay warp-uniform values), one elected
        // lane issues.
        {
            const bool leader = elect_one();
            const uint64_t policy = l2_policy_evict_first();
            int gs = 0;
            uint32_t ph = 0;
            SegIter it;
            it.start(p, block);
            Seg s;
            while (ok && it.next(p, block, s)) {
                const TileRef tr = tile_ref(p, s.tile);
                const void *map = &maps.m[tr.prob];
                for (int i0 = 0; i0 < s.nit; i0 += kGroup) {
                    if (!__all_sync(0xffffffffu, mbar_wait(empty_pk(gs), ph ^ 1, abort_flag, p.status, 1, lim))) { ok = false; break; }
                    // always a whole box of three K blocks: in a short last group the surplus lands in the group's unused
                    // stages (rows beyond the weight read as zeros), and the byte count the barrier expects stays the same
                    if (leader) {
                        mbar_arrive_expect_tx(full_pk(gs), kGroup * Pk<FMT>::kStageBytes);
                        tma_load_3d(sbase + L::pk + gs * kGroup * Pk<FMT>::kStageBytes, map, 0, tr.nt * 4, s.kb0 + i0, full_pk(gs), policy);
                    }
                    if (++gs == kPkG) { gs = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == kMmaWarp || warp == kMmaWarp2) {
        // ---------------- MMA issuers (warp-uniform, one elected lane issues) + epilogue (whole warp) ----------------
        const bool leader = elect_one();
        const int k16 = warp == kMmaWarp ? 0 : 1;
        constexpr uint32_t idesc = instr_desc_bf16_f32(BN, NB, /*a_mn_major=*/true, /*b_mn_major=*/false);
        const uint64_t a_desc0 = smem_desc_noswizzle(sbase + L::a, kA_LBO, kA_SBO);
        const uint64_t b_desc0 = smem_desc_noswizzle(sbase + L::b, kB_LBO, kB_SBO);
        const uint32_t a_lo0 = (uint32_t)a_desc0 + (uint32_t)k16 * ((2 * kA_LBO) >> 4), a_hi = (uint32_t)(a_desc0 >> 32);
        const uint32_t b_lo0 = (uint32_t)b_desc0 + (uint32_t)k16 * ((2 * kB_LBO) >> 4), b_hi = (uint32_t)(b_desc0 >> 32);
        auto mk = [](uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; };
        const uint32_t d_tmem = tmem_base + (uint32_t)(k16 * NB);
        grid_dep_wait();   // the epilogues touch scratch and outputs
        if (p.ranks > 1 && blockIdx.x == 0 && warp == kMmaWarp && lane == 0) *p.expected = *p.expected + p.launch_arrivals;
        int gt = 0, seg_idx = 0;
        uint32_t ph = 0;
        SegIter it;
        it.start(p, block);
        Seg s;
        for (; it.next(p, block, s); ++seg_idx) {
            if (ok) {
                for (int i0 = 0; i0 < s.nit; i0 += kGroup) {
                    const int r = min(kGroup, s.nit - i0);
                    if (!__all_sync(0xffffffffu, mbar_wait(full_ab(gt), ph, abort_flag, p.status, 2, lim))) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a_lo = a_lo0 + (uint32_t)gt * ((kGroup * kAStageBytes) >> 4);
                    const uint32_t b_lo = b_lo0 + (uint32_t)gt * ((kGroup * L::kBStageBytes) >> 4);
#pragma unroll
                    for (int j = 0; j < kGroup; ++j) {
                        if (j < r && leader)
                            mma_bf16_ss(d_tmem, mk(a_lo + (uint32_t)((j * kAStageBytes) >> 4), a_hi),
                                        mk(b_lo + (uint32_t)((j * L::kBStageBytes) >> 4), b_hi), idesc, i0 > 0 || j > 0);
                    }
                    if (leader) mma_commit(empty_ab(gt));
                    if (++gt == kAbGroups) { gt = 0; ph ^= 1; }
                }
                if (ok && leader) mma_commit(accum_bar);
            }
            __syncwarp();
            ok = stream_epilogue<FMT, NB>(p, ectx, s, seg_idx, ok);
            tc_fence_after_sync();
        }
    } else {
        // ---------------- expand warps: packed -> bf16 operands; warps 5..7 and 9..11 also run the epilogues ----------------
        const int ew = (warp >> 2) * 3 + (warp & 3) - 1;
        const int triplet = ew / kGroup, member = ew % kGroup;
        const bool in_epi = warp >= kEpiWarp0;
        constexpr int kActChunks = NB / 8;
        uint4 act_regs[kActChunks];
        int64_t act_off[kActChunks];
#pragma unroll
        for (int j = 0; j < kActChunks; ++j) {
            const int c = j * 32 + lane;
            act_off[j] = act_chunk_base(p, c % NB, c / NB);
        }
        const int act_step = act_chunk_step(p);
        const int64_t chunk_step = p.a_row_major ? (int64_t)NB * p.K : (int64_t)(NB / 32) * p.Kt * 1024;   // one row chunk further
        grid_dep_wait();
        if (p.wait_arrived) {
            int good = 1;
            if (lane == 0) good = peer_wait(p, abort_flag, 6) ? 1 : 0;
            if (!__shfl_sync(0xffffffffu, good, 0)) ok = false;
        }
        // Two cursors over this block's segments: `cur` follows the groups this warp works on (with the number of groups
        // before the segment, cur_g0), `epi` the epilogues it has run. The block's groups are numbered across segments; the
        // triplet of warps `triplet` takes every third one, and inside a group this warp expands stage `member`.
        SegIter cur_it;
        cur_it.start(p, block);
        int cur_g0 = 0, cur_ng = 0, cur_si = -1;
        Seg cur = {0, 0, 0, 1, 0, 0};
        const uint16_t *cur_act = p.a;   // activations of K-block 0 of the current segment's row chunk
        bool more = true;
        // advances `cur` to the segment that holds group G; false once the block's work ends (rare path, kept out of the loop body)
        auto locate_slow = [&](int G) {
            while (G >= cur_g0 + cur_ng) {
                cur_g0 += cur_ng;
                if (!cur_it.next(p, block, cur)) {
                    cur_ng = 0;
                    return false;
                }
                cur_ng = (cur.nit + kGroup - 1) / kGroup;
                ++cur_si;
                cur_act = p.a + (int64_t)(cur.tile / p.tstart[p.nprob]) * chunk_step + (int64_t)cur.kb0 * act_step;
            }
            return true;
        };
        const bool coherent_loads = p.wait_arrived != nullptr;   // activations written by other GPUs during this kernel's life
        auto load_act = [&](int G) {   // activations of this warp's stage of group G (nothing if the group is too short)
            const int st = (G - cur_g0) * kGroup + member;
            if (st >= cur.nit) return;
            const uint16_t *base = cur_act + (int64_t)st * act_step;
            if (coherent_loads) {
#pragma unroll
                for (int j = 0; j < kActChunks; ++j) act_regs[j] = __ldcg(reinterpret_cast<const uint4 *>(base + act_off[j]));
            } else {
#pragma unroll
                for (int j = 0; j < kActChunks; ++j) act_regs[j] = __ldg(reinterpret_cast<const uint4 *>(base + act_off[j]));
            }
        };
        SegIter epi_it;
        epi_it.start(p, block);
        int epi_done = 0;
        auto epilogues_up_to = [&](int upto) {
            while (epi_done < upto) {
                Seg s;
                if (!epi_it.next(p, block, s)) break;
                ok = stream_epilogue<FMT, NB>(p, ectx, s, epi_done, ok);
                ++epi_done;
            }
        };
        const int lane_pk = lane * (FMT == TTB_BFLOAT8_B ? 16 : 8);
        const int lane_a = ((lane & 15) >> 3) * kA_LBO + (lane >> 4) * 2 * kA_SBO + (lane & 7) * 16;
        int G = triplet;
        // ring positions of group G, kept incrementally: G advances by three
        int gs = G % kPkG, gt = G % kAbGroups;
        uint32_t phs = (uint32_t)(G / kPkG) & 1u, pht = (uint32_t)(G / kAbGroups) & 1u;
        more = ok && locate_slow(G);
        if (more) load_act(G);
        while (true) {
            // every earlier segment is finished before any stage of this one is touched; at the end, whatever is left
            if (in_epi) epilogues_up_to(more && ok ? cur_si : (1 << 30));
            if (!more || !ok) break;
            const bool present = (G - cur_g0) * kGroup + member < cur.nit;
            const int sl = gs * kGroup + member, t = gt * kGroup + member;
            int good = 1;
            if (lane == 0)
                good = mbar_wait(empty_ab(gt), pht ^ 1, abort_flag, p.status, 3, lim) && mbar_wait(full_pk(gs), phs, abort_flag, p.status, 4, lim);
            good = __shfl_sync(0xffffffffu, good, 0);
            if (!good) { ok = false; continue; }   // (the top of the loop still runs this warp's share of the epilogues)
            if (present) {
                const uint8_t *pst = smem + L::pk + sl * Pk<FMT>::kStageBytes;
                uint8_t *const ast = smem + L::a + t * kAStageBytes + lane_a;
                uint8_t *const bst = smem + L::b + t * L::kBStageBytes;
                uint32_t Es[8];
                uint32_t codes[8][4];
#pragma unroll
                for (int rr = 0; rr < 8; ++rr) {
                    const uint8_t *tb = pst + (rr >> 1) * TB;
                    Es[rr] = tb[(rr & 1) * 32 + lane];
                    if (FMT == TTB_BFLOAT8_B) {
                        const uint4 cv = *reinterpret_cast<const uint4 *>(tb + 64 + (rr & 1) * 512 + lane_pk);
                        codes[rr][0] = cv.x; codes[rr][1] = cv.y; codes[rr][2] = cv.z; codes[rr][3] = cv.w;
                    } else {
                        const uint2 cv = *reinterpret_cast<const uint2 *>(tb + 64 + (rr & 1) * 256 + lane_pk);
                        codes[rr][0] = cv.x; codes[rr][1] = cv.y; codes[rr][2] = 0; codes[rr][3] = 0;
                    }
                }
                uint32_t emax = Es[0];
#pragma unroll
                for (int rr = 1; rr < 8; ++rr) emax = max(emax, Es[rr]);
                auto expand_stage = [&](auto big) {
#pragma unroll
                    for (int rr = 0; rr < 8; ++rr) {
                        uint32_t vals[8];
                        expand_row<FMT, decltype(big)::value>(codes[rr], Es[rr], vals);
                        uint8_t *dst = ast + (rr & 1) * 2 * kA_LBO + (rr >> 1) * 4 * kA_SBO;
                        *reinterpret_cast<uint4 *>(dst) = make_uint4(vals[0], vals[1], vals[2], vals[3]);
                        *reinterpret_cast<uint4 *>(dst + kA_SBO) = make_uint4(vals[4], vals[5], vals[6], vals[7]);
                    }
                };
                if (__any_sync(0xffffffffu, emax > 127u))
                    expand_stage(std::true_type{});
                else
                    expand_stage(std::false_type{});
#pragma unroll
                for (int j = 0; j < kActChunks; ++j) {
                    const int c = j * 32 + lane;
                    const int m = c % NB, kc = c / NB;
                    *reinterpret_cast<uint4 *>(bst + (m >> 3) * kB_SBO + kc * kB_LBO + (m & 7) * 16) = act_regs[j];
                }
                fence_proxy_async_smem();
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(full_ab(gt));
                mbar_arrive(empty_pk(gs));
            }
            G += kExpandWarps / kGroup;
            gs += kExpandWarps / kGroup;
            if (gs >= kPkG) { gs -= kPkG; phs ^= 1u; }
            gt += kExpandWarps / kGroup;
            if (gt >= kAbGroups) { gt -= kAbGroups; pht ^= 1u; }
            more = G < cur_g0 + cur_ng || locate_slow(G);
            if (more) load_act(G);
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <int FMT, int NB>
int32_t launch_one(const DecodeArgs &p, const WeightMaps &maps, bool overlap, cudaStream_t stream) {
    constexpr int smem_bytes = StreamLayout<FMT, NB>::total + 128;
    static_assert(smem_bytes <= 232448, "shared memory budget");
    static bool configured[64] = {};
    int dev = 0;
    TTB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        TTB_CUDA_TRY(cudaFuncSetAttribute(matmul_decode_stream_kernel<FMT, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)p.sk_grid);
    cfg.blockDim = dim3(kThreadsDecode);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    TTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, matmul_decode_stream_kernel<FMT, NB>, p, maps));
    TTB_LAUNCH_CHECK("matmul_decode_stream");
    return TTB_OK;
}

}  // namespace


// Tensor maps of the launch's weights. cuTensorMapEncodeTiled is reached through the runtime's driver entry point (no link
// against the driver library).
int32_t make_weight_maps(const DecodeArgs &p, int fmt, WeightMaps &maps, int group) {
    using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        TTB_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return fail(TTB_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const cuuint64_t tile_bytes = (cuuint64_t)bfp_tile_bytes(fmt);
    for (int j = 0; j < p.nprob; ++j) {
        const cuuint64_t Nt = (cuuint64_t)(p.Nv[j] / 32), Kt = (cuuint64_t)p.Kt;
        const cuuint64_t dims[3] = {tile_bytes / 8, Nt, Kt};
        const cuuint64_t strides[2] = {tile_bytes, Nt * tile_bytes};
        const cuuint32_t box[3] = {(cuuint32_t)(tile_bytes / 8), 4, (cuuint32_t)group};   // `group` K blocks = one group of stages
        const cuuint32_t estr[3] = {1, 1, 1};
        const CUresult r = encode(&maps.m[j], CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<uint8_t *>(p.wv[j]), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(TTB_E_CUDA, "cuTensorMapEncodeTiled failed with %d for weight %d", (int)r, j);
    }
    for (int j = p.nprob; j < TTB_MAX_GROUP; ++j) maps.m[j] = maps.m[0];
    return TTB_OK;
}

static int32_t tensor_map_encoder(void **out) {
    static void *encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        TTB_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) return fail(TTB_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        encode = fn;
    }
    *out = encode;
    return TTB_OK;
}

int32_t make_act_map(const DecodeArgs &p, int64_t rows, ActMap &map, int group) {
    using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    void *fn = nullptr;
    if (int32_t rc = tensor_map_encoder(&fn)) return rc;
    EncodeFn encode = reinterpret_cast<EncodeFn>(fn);
    CUresult r;
    const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    void *base = const_cast<uint16_t *>(p.a);
    if (p.a_row_major) {
        // [rows][K]: 16 values, rows, 16-column chunks
        const cuuint64_t dims[3] = {16, (cuuint64_t)rows, (cuuint64_t)(p.K / 16)};
        const cuuint64_t strides[2] = {(cuuint64_t)p.K * 2, 32};
        const cuuint32_t box[3] = {16, 32, (cuuint32_t)(2 * group)};
        r = encode(&map.m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    } else {
        // tiles of 2048 bytes in (row tile, K tile) order; inside: 16 values, 16 face rows, upper / lower faces, left / right faces
        const cuuint64_t dims[5] = {16, 16, 2, 2, (cuuint64_t)((rows / 32) * p.Kt)};
        const cuuint64_t strides[4] = {32, 1024, 512, 2048};
        const cuuint32_t box[5] = {16, 16, 2, 2, (cuuint32_t)group};
        r = encode(&map.m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    if (r != CUDA_SUCCESS) return fail(TTB_E_CUDA, "cuTensorMapEncodeTiled failed with %d for the activation", (int)r);
    return TTB_OK;
}

int32_t launch_decode_stream(const DecodeArgs &p, int fmt, int nb, bool overlap, cudaStream_t stream) {
    WeightMaps maps;
    if (int32_t rc = make_weight_maps(p, fmt, maps)) return rc;
#define TTB_STREAM(F, B) return launch_one<F, B>(p, maps, overlap, stream)
    if (fmt == TTB_BFLOAT8_B) {
        if (nb == 32) TTB_STREAM(TTB_BFLOAT8_B, 32);
        if (nb == 64) TTB_STREAM(TTB_BFLOAT8_B, 64);
        TTB_STREAM(TTB_BFLOAT8_B, 128);
    }
    if (nb == 32) TTB_STREAM(TTB_BFLOAT4_B, 32);
    if (nb == 64) TTB_STREAM(TTB_BFLOAT4_B, 64);
    TTB_STREAM(TTB_BFLOAT4_B, 128);
#undef TTB_STREAM
}

}  // namespace ttb
