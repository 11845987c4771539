// Streamed decode matmul for bfloat8_b / bfloat4_b weights and 32 or 64 activation rows per block (one or two tile rows,
// template parameter NB), weight operand through tensor memory, persistent form:
//   out_j[rows, N_j] = act(a[rows, K] x W_j[K, N_j] + bias_j)   for up to four weights W_j that share the activation,
// optionally several such stages in one launch, the product of a gated pair, and the all-gather of the first result.
//
// Same work decomposition as matmul_decode_stream.cu (one list of 128-column tiles over all weights of the launch, at most
// one persistent block per SM working through (tile, K range) segments, partial sums of shared tiles exchanged through
// scratch, optional store of finished tiles into the other ranks' copies), "swap-AB": the MMA's M dimension (128 TMEM
// lanes) runs over weight columns, its N dimension over the activation rows.
//
// Why tensor memory: expanded to bf16 a weight is two bytes; writing it to shared memory and letting the MMA fetch it
// back costs four bytes of shared-memory traffic per packed byte that HBM delivers. Here a packed tile crosses shared
// memory once (tensor-map copy in, ldmatrix out) and the bf16 values go registers -> tensor memory -> MMA:
//   * ldmatrix.m16n16.trans.b8 reads a 16x16 face of 8-bit codes transposed, so that a lane holds four consecutive K
//     values of one weight column - the order the MMA's A operand wants (TMEM lane = column n, TMEM column = K pair);
//   * the codes become bf16 with one byte-permute, one mask and one packed multiply per pair ((sign << 15) | mantissa is,
//     read as bf16, the weight divided by 2^E); the per-row powers of two come from a warp-wide table of the tile's 64
//     exponents (one pair per lane, fetched by shuffle);
//   * tcgen05.st.16x256b has exactly the fragment layout ldmatrix produced; tcgen05.mma takes A from tensor memory and
//     the activations (B) from shared memory.
//
// Roles (20 warps). A warp can only touch the 32 TMEM lanes of its quadrant (warp % 4) = one of the four packed tiles of
// a K block, so the expand warps 0..11 form three teams of four; team t expands every third group of four K blocks, two
// tiles at a time. They do nothing else: no global loads, no epilogue. Warps 12..15 run the epilogues (one per TMEM lane
// quadrant) on one of two accumulator sets while the MMAs of the next segment fill the other. Warp 16 streams the packed
// tiles with one tensor-map copy per group; warp 19 streams the activations of the same group with another tensor-map
// copy that delivers them in the MMA's swizzled K-major operand layout; warps 17 and 18 issue the MMAs, taking alternate
// pairs of groups, each into its own accumulator. These four warps run warp-uniform: all lanes walk the work list, one
// elected lane issues, so that addresses and descriptors are uniform-datapath values (with a single active lane every
// MMA and copy paid for moving its operands between register files: 17 % of the kernel's time).
// Three rings: packed tiles in shared memory (released as soon as they are expanded: the next copy from HBM starts
// then), expanded weights in tensor memory and activations in shared memory (released by the commit of the pair's MMAs).
// Every wait is bounded; a wait that runs out raises a status word instead of hanging.
#include "decode_common.cuh"

namespace ttb {

#ifdef TTB_TIMELINE
// Scratch instrumentation (never part of the product build): clock stamps of block 0's roles per group of stages.
__device__ long long g_tl[12][2048];
#define TL(role, g) do { if (blockIdx.x == 0 && (g) < 2048) g_tl[role][g] = clock64(); } while (0)
#else
#define TL(role, g) do { } while (0)
#endif

namespace {

using namespace ptx;

constexpr int BN = 128;  // weight columns per tile (MMA M, TMEM lanes)
constexpr int BK = 32;   // K per stage: one row of four packed tiles
constexpr int kGroup = 4;                      // stages (K blocks) per group: one barrier round trip and one copy of each kind per group
constexpr int kTeams = 3;                      // expand teams of four warps
constexpr int kExpandWarps = 4 * kTeams;       // warps 0..11; quadrant = warp % 4, team = warp / 4
constexpr int kEpiWarp0 = kExpandWarps;        // warps 12..15
constexpr int kEpiThreads = 128;
constexpr int kProducerWarp = kEpiWarp0 + 4, kMmaWarp = kProducerWarp + 1, kLoaderWarp = kProducerWarp + 3;   // two MMA issuers
constexpr int kThreads = 32 * (kLoaderWarp + 1);
// (NB, a template parameter below: activation rows per block = the MMA's N, 32 or 64 - one or two tile rows)
constexpr int kAColsPerStage = BK / 2;         // TMEM columns of one expanded stage (two bf16 per column)
constexpr uint32_t kB_SBO = 256;               // activations: 32-byte rows, eight rows per swizzle atom

template <int FMT, int NB>
struct Layout {
    static constexpr int kTile = FMT == TTB_BFLOAT8_B ? kBfp8TileBytes : kBfp4TileBytes;
    static constexpr int kStageBytes = 4 * kTile;                  // 4352 / 2304
    static constexpr int kRing = 6;                                // groups whose activations / expanded weights are in flight
    // Packed tiles in flight: the copies from HBM need ~100 KB per SM under way to keep the memory system busy, on top of
    // the groups that sit in shared memory while they are expanded, so this ring is deeper than the one above.
    static constexpr int kWRing = FMT == TTB_BFLOAT8_B ? (NB == 32 ? 9 : 6) : (NB == 32 ? 15 : 12);
    static constexpr int kBRowStage = 32 * BK * 2;                 // activations of one K block, one tile row (32 rows): 2 KiB
    static constexpr int kBStageBytes = NB * BK * 2;               // ... of the block's NB rows (the tile rows lie one behind the other per group)
    static constexpr int pk = 0;
    static constexpr int b = pk + kWRing * kGroup * kStageBytes;   // (a multiple of 256: the swizzled operand needs it)
    static constexpr int stage = b + kRing * kGroup * kBStageBytes;   // [NB x 128] bf16 tiled slab for the gather epilogue
    static constexpr int bars = stage + NB * BN * 2;
    // full_b[kRing], full_a[kRing], empty[kRing] (one per pair of groups used), acc_full[2], acc_empty[2], full_w[kWRing], w_empty[kWRing]
    static constexpr int nbars = 3 * kRing + 4 + 2 * kWRing;
    static constexpr int misc = bars + 8 * nbars;                  // tmem base, abort flag, last-block flag, two accumulator-ready flags
    static constexpr int total = misc + 32;
    // Issuing costs a thread ~46 cycles per MMA and ~300 per commit, whatever the MMA's size. Two issuing threads take
    // alternate pairs of groups (six stages, twelve MMAs, one commit that frees the pair's ring slots), each into its own
    // accumulator, so that no ordering between the two is needed; the epilogue adds the accumulators.
    static constexpr int kAccs = 2;
    // Accumulator sets: two for one tile row per block (the epilogue of a segment runs while the next segment's MMAs fill the
    // other set); with two tile rows tensor memory holds one set next to the ring of expanded weights.
    static constexpr int kSets = NB == 32 ? 2 : 1;
    static constexpr int kAccCols = kSets * kAccs * NB;
    static constexpr int kACol0 = kAccCols;                        // the A ring follows them
    static constexpr int kTmemColsUsed = kAccCols + kRing * kGroup * kAColsPerStage;
    static constexpr int kTmemCols = kTmemColsUsed <= 256 ? 256 : 512;
    static_assert(kTmemColsUsed <= 512, "tensor memory budget");
    static_assert(b % 256 == 0 && kBStageBytes % 1024 == 0, "alignment of the swizzled activation operand");
    // The teams wait on the ring barriers with different phase parities, which is only right while a waiter is at most
    // one phase behind, i.e. while the ring has at least as many groups as there are teams.
    static_assert(kTeams <= kRing && kRing % 2 == 0 && kTeams <= kWRing, "ring shorter than the number of teams");
    // ... and only while every team meets every phase of the barriers it waits on: a team takes every kTeams-th group, so
    // the rings' lengths must be multiples of kTeams (with a ring of four and three teams, a team came back to a pair of
    // slots two phases later; when one MMA issuer lagged behind the other, its parity wait passed on the stale phase and
    // the team overwrote expanded weights that had not been multiplied yet).
    static_assert(kRing % kTeams == 0 && kWRing % kTeams == 0, "every team must see every phase of a ring slot");
};

struct Seg {
    int tile, kb0, nit, contributors, slot0, slot;
};

__device__ __forceinline__ int unit_begin(const DecodeArgs &p, int b) { return b * p.sk_q + min(b, p.sk_r); }
__device__ __forceinline__ int block_of_unit(const DecodeArgs &p, int u) {
    const int big = p.sk_r * (p.sk_q + 1);
    return u < big ? u / (p.sk_q + 1) : p.sk_r + (u - big) / p.sk_q;
}

// A block's segments in order (the plan is described in matmul_decode_stream.cu: pieces taken round by round, or whole
// tiles round by round followed by the block's share of the evenly streamed remainder).
struct SegIter {
    int w, u, u_end;
    __device__ __forceinline__ void start(const DecodeArgs &p, int block) {
        if (block < p.sk_grid) {
            w = 0;
            u = unit_begin(p, block);
            u_end = unit_begin(p, block + 1);
        } else {   // a stage planned for fewer blocks than the launch has
            w = p.sk_waves;
            u = u_end = 0;
        }
    }
    __device__ __forceinline__ bool next(const DecodeArgs &p, int block, Seg &s) {
        while (w < p.sk_waves) {
            const int q = w * p.sk_grid + block;
            ++w;
            if (q < p.sk_rem_tile0) {
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

// A launch runs a sequence of stages, each what one ttb_matmul_multi call describes. The persistent blocks walk the stages
// one after the other without meeting in between: the weight stream, the expansion and the MMAs continue across stage
// borders, and a stage that consumes what an earlier one produced (or what the ranks gathered) holds only its activation
// copies until that is complete.
template <int S>
struct alignas(64) Sequence {
    int n, grid;
    int *sync;    // zero between launches: [0] blocks that have finished the launch, [1 + s] tiles of stage s stored (if counted)
    DecodeArgs st[S];
    WeightMaps maps[S];
    ActMap amap[S];
};

// A block's segments over all stages, in order.
template <int S>
struct WorkIter {
    int si;
    SegIter it;
    __device__ __forceinline__ void start(const Sequence<S> &q, int block) {
        si = 0;
        it.start(q.st[0], block);
    }
    __device__ __forceinline__ bool next(const Sequence<S> &q, int block, Seg &s) {
        while (true) {
            if (it.next(q.st[S == 1 ? 0 : si], block, s)) return true;
            if (S == 1 || si + 1 >= q.n) return false;
            ++si;
            it.start(q.st[si], block);
        }
    }
};

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

__device__ __forceinline__ void ldmatrix_x2_trans_b8(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void tmem_st_16x256b(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("tcgen05.st.sync.aligned.16x256b.x1.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}

__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
    __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&a), *reinterpret_cast<__nv_bfloat162 *>(&b));
    return *reinterpret_cast<uint32_t *>(&v);
}
// Four codes (consecutive K of one column) -> two packed bf16 pairs, each multiplied by its pair of row scales.
__device__ __forceinline__ void expand4(uint32_t codes, uint32_t s01, uint32_t s23, uint32_t &o01, uint32_t &o23) {
    o01 = mul2(__byte_perm(codes, 0u, 0x1100u) & 0x807f807fu, s01);
    o23 = mul2(__byte_perm(codes, 0u, 0x3322u) & 0x807f807fu, s23);
}

// One packed tile (1088 bytes at shared address `tile`) -> the 32 TMEM lanes of this warp's quadrant, 16 columns at a_col.
// BIG: some exponent of the tile exceeds 127 (a row maximum of 2 or more), whose power of two needs a second factor.
template <bool BIG>
__device__ __forceinline__ void expand_tile(uint32_t tile, uint32_t a_col, uint32_t ld_off, uint32_t eh, int sh0) {
    const uint32_t my_scale = (__vminu2(eh, 0x007f007fu) + 0x007f007fu) << 7;   // 2^min(E, 127) per half
    const uint32_t my_t = BIG ? (__vmaxu2(__vminu2(eh, 0x00fe00feu), 0x007f007fu) << 7) : 0u;
    uint32_t top[4], bot[4];
    ldmatrix_x2_trans_b8(tile + ld_off, top);         // faces 0 (left) and 1 (right): K 0..15
    ldmatrix_x2_trans_b8(tile + ld_off + 512u, bot);  // faces 2 and 3: K 16..31
#pragma unroll
    for (int f = 0; f < 4; ++f) {
        // face f = 2 * kh + nh; registers {2*nh, 2*nh+1} of the kh-th load: columns lane/4 and lane/4 + 8
        const uint32_t c0 = (f >> 1) ? bot[2 * (f & 1)] : top[2 * (f & 1)];
        const uint32_t c1 = (f >> 1) ? bot[2 * (f & 1) + 1] : top[2 * (f & 1) + 1];
        const uint32_t s01 = __shfl_sync(0xffffffffu, my_scale, 8 * f + sh0);
        const uint32_t s23 = __shfl_sync(0xffffffffu, my_scale, 8 * f + sh0 + 1);
        uint32_t o[4];
        expand4(c0, s01, s23, o[0], o[1]);
        expand4(c1, s01, s23, o[2], o[3]);
        if (BIG) {
            const uint32_t t01 = __shfl_sync(0xffffffffu, my_t, 8 * f + sh0);
            const uint32_t t23 = __shfl_sync(0xffffffffu, my_t, 8 * f + sh0 + 1);
            o[0] = mul2(o[0], t01); o[1] = mul2(o[1], t23); o[2] = mul2(o[2], t01); o[3] = mul2(o[3], t23);
        }
        // TMEM lanes 32*quad + 16*nh + {lane/4, lane/4 + 8}; columns: stage base + 8*kh + 2*(lane%4) + {0, 1}
        tmem_st_16x256b(a_col + ((uint32_t)((f & 1) * 16) << 16) + (uint32_t)((f >> 1) * 8), o[0], o[1], o[2], o[3]);
    }
}
// Two tiles at once (the common case: no exponent above 127): the transposing loads of both go out first and the faces
// are expanded alternately, so that one tile's shuffles and stores wait behind the other's arithmetic.
__device__ __forceinline__ void expand_pair(uint32_t tile0, uint32_t tile1, uint32_t a_col0, uint32_t a_col1, uint32_t ld_off, uint32_t eh0,
                                            uint32_t eh1, int sh0) {
    const uint32_t scale0 = (__vminu2(eh0, 0x007f007fu) + 0x007f007fu) << 7, scale1 = (__vminu2(eh1, 0x007f007fu) + 0x007f007fu) << 7;
    uint32_t top0[4], bot0[4], top1[4], bot1[4];
    ldmatrix_x2_trans_b8(tile0 + ld_off, top0);
    ldmatrix_x2_trans_b8(tile0 + ld_off + 512u, bot0);
    ldmatrix_x2_trans_b8(tile1 + ld_off, top1);
    ldmatrix_x2_trans_b8(tile1 + ld_off + 512u, bot1);
#pragma unroll
    for (int f = 0; f < 4; ++f) {
        const uint32_t p01 = __shfl_sync(0xffffffffu, scale0, 8 * f + sh0), p23 = __shfl_sync(0xffffffffu, scale0, 8 * f + sh0 + 1);
        const uint32_t q01 = __shfl_sync(0xffffffffu, scale1, 8 * f + sh0), q23 = __shfl_sync(0xffffffffu, scale1, 8 * f + sh0 + 1);
        const uint32_t c0 = (f >> 1) ? bot0[2 * (f & 1)] : top0[2 * (f & 1)], c1 = (f >> 1) ? bot0[2 * (f & 1) + 1] : top0[2 * (f & 1) + 1];
        const uint32_t d0 = (f >> 1) ? bot1[2 * (f & 1)] : top1[2 * (f & 1)], d1 = (f >> 1) ? bot1[2 * (f & 1) + 1] : top1[2 * (f & 1) + 1];
        uint32_t o[4], w[4];
        expand4(c0, p01, p23, o[0], o[1]);
        expand4(d0, q01, q23, w[0], w[1]);
        expand4(c1, p01, p23, o[2], o[3]);
        expand4(d1, q01, q23, w[2], w[3]);
        const uint32_t off = ((uint32_t)((f & 1) * 16) << 16) + (uint32_t)((f >> 1) * 8);
        tmem_st_16x256b(a_col0 + off, o[0], o[1], o[2], o[3]);
        tmem_st_16x256b(a_col1 + off, w[0], w[1], w[2], w[3]);
    }
}
__device__ __noinline__ void expand_tile_big(uint32_t tile, uint32_t a_col, uint32_t ld_off, uint32_t eh, int sh0) {
    expand_tile<true>(tile, a_col, ld_off, eh, sh0);
}

// One packed bfloat4_b tile (576 bytes) -> the 32 TMEM lanes of this warp's quadrant. One transposing load covers the whole
// tile: per 16-column half a lane receives two registers - four bytes of even K rows and four of odd K rows, each byte
// the codes of columns 2p (low nibble) and 2p + 1 (high nibble), p = lane / 4. Column 2p goes to TMEM lane p, column 2p + 1
// to TMEM lane p + 8 of the half (the epilogue reads its column index accordingly). (sign << 15) | (mantissa << 4) is the
// weight divided by 2^(E + 4 - ...): the same subnormal trick and the same row scales as for bfloat8_b.
__device__ __forceinline__ void ldmatrix_x2_trans_b8_2(uint32_t addr, uint32_t &a, uint32_t &b, uint32_t &c, uint32_t &d) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}
template <bool BIG>
__device__ __forceinline__ void expand_tile4(uint32_t tile, uint32_t a_col, uint32_t ld_off4, uint32_t eh, int sh0) {
    const uint32_t my_scale = (__vminu2(eh, 0x007f007fu) + 0x007f007fu) << 7;   // 2^min(E, 127) per half
    const uint32_t my_t = BIG ? (__vmaxu2(__vminu2(eh, 0x00fe00feu), 0x007f007fu) << 7) : 0u;
    uint32_t m[2][2];   // [16-column half][even / odd K rows]
    ldmatrix_x2_trans_b8_2(tile + ld_off4, m[0][0], m[0][1], m[1][0], m[1][1]);
#pragma unroll
    for (int nh = 0; nh < 2; ++nh) {
        // [s m m m 0 0 0 0] per byte: columns 2p (from the low nibbles) and 2p + 1 (high nibbles), even and odd K rows
        const uint32_t lo_e = (m[nh][0] << 4) & 0xf0f0f0f0u, lo_o = (m[nh][1] << 4) & 0xf0f0f0f0u;
        const uint32_t hi_e = m[nh][0] & 0xf0f0f0f0u, hi_o = m[nh][1] & 0xf0f0f0f0u;
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) {
            // bytes 2*kh and 2*kh+1 of the registers: K rows 4q..4q+3 of the upper (kh = 0) or lower face
            const int f = 2 * kh + nh;
            const uint32_t s01 = __shfl_sync(0xffffffffu, my_scale, 8 * f + sh0);
            const uint32_t s23 = __shfl_sync(0xffffffffu, my_scale, 8 * f + sh0 + 1);
            const uint32_t sel0 = kh ? 0x6622u : 0x4400u, sel1 = kh ? 0x7733u : 0x5511u;
            uint32_t o[4];
            o[0] = mul2(__byte_perm(lo_e, lo_o, sel0) & 0x80708070u, s01);   // column 2p: K rows (4q, 4q+1)
            o[1] = mul2(__byte_perm(lo_e, lo_o, sel1) & 0x80708070u, s23);   //            K rows (4q+2, 4q+3)
            o[2] = mul2(__byte_perm(hi_e, hi_o, sel0) & 0x80708070u, s01);   // column 2p + 1
            o[3] = mul2(__byte_perm(hi_e, hi_o, sel1) & 0x80708070u, s23);
            if (BIG) {
                const uint32_t t01 = __shfl_sync(0xffffffffu, my_t, 8 * f + sh0);
                const uint32_t t23 = __shfl_sync(0xffffffffu, my_t, 8 * f + sh0 + 1);
                o[0] = mul2(o[0], t01); o[1] = mul2(o[1], t23); o[2] = mul2(o[2], t01); o[3] = mul2(o[3], t23);
            }
            tmem_st_16x256b(a_col + ((uint32_t)(nh * 16) << 16) + (uint32_t)(kh * 8), o[0], o[1], o[2], o[3]);
        }
    }
}
// Two bfloat4_b tiles at once, as expand_pair.
__device__ __forceinline__ void expand_pair4(uint32_t tile0, uint32_t tile1, uint32_t a_col0, uint32_t a_col1, uint32_t ld_off4, uint32_t eh0,
                                             uint32_t eh1, int sh0) {
    const uint32_t scale0 = (__vminu2(eh0, 0x007f007fu) + 0x007f007fu) << 7, scale1 = (__vminu2(eh1, 0x007f007fu) + 0x007f007fu) << 7;
    uint32_t m[2][2], k[2][2];
    ldmatrix_x2_trans_b8_2(tile0 + ld_off4, m[0][0], m[0][1], m[1][0], m[1][1]);
    ldmatrix_x2_trans_b8_2(tile1 + ld_off4, k[0][0], k[0][1], k[1][0], k[1][1]);
#pragma unroll
    for (int nh = 0; nh < 2; ++nh) {
        const uint32_t lo_e = (m[nh][0] << 4) & 0xf0f0f0f0u, lo_o = (m[nh][1] << 4) & 0xf0f0f0f0u;
        const uint32_t hi_e = m[nh][0] & 0xf0f0f0f0u, hi_o = m[nh][1] & 0xf0f0f0f0u;
        const uint32_t ko_e = (k[nh][0] << 4) & 0xf0f0f0f0u, ko_o = (k[nh][1] << 4) & 0xf0f0f0f0u;
        const uint32_t ki_e = k[nh][0] & 0xf0f0f0f0u, ki_o = k[nh][1] & 0xf0f0f0f0u;
#pragma unroll
        for (int kh = 0; kh < 2; ++kh) {
            const int f = 2 * kh + nh;
            const uint32_t p01 = __shfl_sync(0xffffffffu, scale0, 8 * f + sh0), p23 = __shfl_sync(0xffffffffu, scale0, 8 * f + sh0 + 1);
            const uint32_t q01 = __shfl_sync(0xffffffffu, scale1, 8 * f + sh0), q23 = __shfl_sync(0xffffffffu, scale1, 8 * f + sh0 + 1);
            const uint32_t sel0 = kh ? 0x6622u : 0x4400u, sel1 = kh ? 0x7733u : 0x5511u;
            uint32_t o[4], w[4];
            o[0] = mul2(__byte_perm(lo_e, lo_o, sel0) & 0x80708070u, p01);
            w[0] = mul2(__byte_perm(ko_e, ko_o, sel0) & 0x80708070u, q01);
            o[1] = mul2(__byte_perm(lo_e, lo_o, sel1) & 0x80708070u, p23);
            w[1] = mul2(__byte_perm(ko_e, ko_o, sel1) & 0x80708070u, q23);
            o[2] = mul2(__byte_perm(hi_e, hi_o, sel0) & 0x80708070u, p01);
            w[2] = mul2(__byte_perm(ki_e, ki_o, sel0) & 0x80708070u, q01);
            o[3] = mul2(__byte_perm(hi_e, hi_o, sel1) & 0x80708070u, p23);
            w[3] = mul2(__byte_perm(ki_e, ki_o, sel1) & 0x80708070u, q23);
            const uint32_t off = ((uint32_t)(nh * 16) << 16) + (uint32_t)(kh * 8);
            tmem_st_16x256b(a_col0 + off, o[0], o[1], o[2], o[3]);
            tmem_st_16x256b(a_col1 + off, w[0], w[1], w[2], w[3]);
        }
    }
}
__device__ __noinline__ void expand_tile4_big(uint32_t tile, uint32_t a_col, uint32_t ld_off4, uint32_t eh, int sh0) {
    expand_tile4<true>(tile, a_col, ld_off4, eh, sh0);
}

struct EpiCtx {
    uint8_t *smem;
    uint32_t tmem_base, acc_full0, acc_empty0;
    volatile int *abort_flag;
    volatile int *last_flag;
    long long lim;
};

constexpr int kPartialsUpTo = 1;   // plain partial tiles (fixed order) only on request: measured ~2 us per launch slower than the reductions even for two sharers

// Epilogue of segment `seg_idx`, run by warps 12..15 together. Always runs through the same barriers, also after a wait
// that ran out (then it moves no data), so that the four warps never part ways at a named barrier.
template <int FMT, int NB>
__device__ __forceinline__ bool epilogue(const DecodeArgs &p, const EpiCtx c, const Seg s, const int seg_idx, const int g0, bool ok, int *done_counter) {
    using L = Layout<FMT, NB>;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tid = threadIdx.x - 32 * kEpiWarp0;
    const int quad = warp & 3;
    const int buf = seg_idx % L::kSets;
    const uint32_t acc_full = c.acc_full0 + 8u * buf, acc_empty = c.acc_empty0 + 8u * buf;
    // one thread waits for the accumulator; the other 127 sleep in a hardware barrier instead of polling
    volatile int *const ready = c.last_flag + 1 + buf;
    if (tid == 0) *ready = (ok && mbar_wait(acc_full, (uint32_t)((seg_idx / L::kSets) & 1), c.abort_flag, p.status, 15, c.lim)) ? 1 : 0;
    asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
    const bool eok = *ready != 0;
    if (tid == 0) { TL(5, seg_idx * 8); }
    tc_fence_after_sync();
    const TileRef tr = tile_ref(p, s.tile);
    const int64_t row0 = (int64_t)tr.rchunk * NB;
    // Which weight column this thread's TMEM lane holds. bfloat8_b: the lane's own. bfloat4_b: a code byte carries two
    // neighbouring columns, and the transposing load hands the even one to lanes 0..7 and the odd one to lanes 8..15 of
    // every 16-lane half (expand_tile4).
    const int col_in_quad = FMT == TTB_BFLOAT8_B ? lane : (lane & 16) + ((lane & 7) << 1) + ((lane >> 3) & 1);
    const int64_t n = (int64_t)tr.nt * BN + quad * 32 + col_in_quad;
    // (the last tile of a weight may hold fewer than 128 columns: no column beyond N is stored)
#define TTB_COL_OK (n < p.Nv[tr.prob])
    // (gated pair: both weights' tiles lead to the one product tensor, which takes the first weight's place)
    const bool gathered = p.ranks > 1 && (tr.prob == 0 || p.gated);
    const int gate_pair = tr.rchunk * p.tstart[1] + tr.nt;
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
    const uint32_t t_acc = c.tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * L::kAccs * NB);
    // Which issuers had a group in this segment: issuer h owns the groups G (numbered over the block's whole work, g0 =
    // this segment's first) with (G / 2) % 2 == h. Three consecutive groups always touch both.
    const int ng = (s.nit + kGroup - 1) / kGroup;
    bool used[L::kAccs];
#pragma unroll
    for (int h = 0; h < L::kAccs; ++h) {
        used[h] = ng >= 3;
        for (int G = g0; G < g0 + min(ng, 2); ++G) used[h] = used[h] || ((G >> 1) & 1) == h;
    }
    auto read_accumulator = [&](int col0, float (&v)[16]) {   // sum of the segment's accumulators, 16 rows of this lane's column
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.0f;
#pragma unroll
        for (int a = 0; a < L::kAccs; ++a) {
            if (used[a]) {
                uint32_t r[16];
                tmem_ld16(t_acc + (uint32_t)(a * NB + col0), r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] += __uint_as_float(r[j]);
            }
        }
    };
    auto release_accumulator = [&]() {
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty);
    };
    bool finished = contributors == 1;
    if (contributors > 1) {
        // phase 1: hand this block's share over (partial tile or reductions), then learn whether it arrived last
        if (eok) {
#pragma unroll
            for (int cc = 0; cc < NB / 16; ++cc) {
                const int col0 = cc * 16;
                float v[16];
                read_accumulator(col0, v);
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
        release_accumulator();
        if (tid == 0) { TL(5, seg_idx * 8 + 1); }
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (tid == 0) { TL(5, seg_idx * 8 + 2); }
        if (tid == 0) {
            *c.last_flag = (atomicAdd(p.counters + s.tile, 1) == contributors - 1) ? 1 : 0;
            __threadfence();   // acquire side: the other blocks' partial sums, published before their tickets, are visible to
                               // every thread that passes the next barrier
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        finished = *c.last_flag != 0;
        if (tid == 0) { TL(5, seg_idx * 8 + 3); }
    }
    // phase 2: whoever holds the complete sum - the only block of an unshared tile, or the last arriver - finishes the tile
    if (finished && (eok || contributors > 1)) {
#pragma unroll
        for (int cc = 0; cc < NB / 16; ++cc) {
            const int col0 = cc * 16;
            float v[16];
            if (contributors == 1) {
                read_accumulator(col0, v);
            } else if (partials) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                // up to three blocks' partials per round: all loads of a round are issued before the first add; the adds
                // stay in block order
#pragma unroll 1
                for (int c0 = 0; c0 < contributors; c0 += 3) {
                    const float4 *src = reinterpret_cast<const float4 *>(
                        p.partial + ((int64_t)(s.slot0 + c0) * BN + quad * 32 + lane) * NB + col0);
                    constexpr int64_t kSlot = (int64_t)BN * NB / 4;   // float4 per slot
                    const int cnt = min(3, contributors - c0);
                    float4 x0[4], x1[4], x2[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        x0[j] = __ldcg(src + j);
                        x1[j] = cnt > 1 ? __ldcg(src + kSlot + j) : make_float4(0.f, 0.f, 0.f, 0.f);
                        x2[j] = cnt > 2 ? __ldcg(src + 2 * kSlot + j) : make_float4(0.f, 0.f, 0.f, 0.f);
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
            if (!p.gated) {
                if (TTB_COL_OK) finish_and_store<NB>(p, ov, v, row0, col0, n, stage);
            } else {
                // gated pair: bias (and, for the first weight, the activation) in fp32, left for whoever finishes the pair
                const float bias = (ov.bias && TTB_COL_OK) ? bias_at(ov.bias, n) : 0.0f;
                float4 *dst = reinterpret_cast<float4 *>(p.gate + ((int64_t)(gate_pair * 2 + tr.prob) * BN + quad * 32 + lane) * NB + col0);
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = tr.prob == 0 ? apply_activation(v[j] + bias, p.act) : v[j] + bias;
#pragma unroll
                for (int j = 0; j < 4; ++j) __stcg(dst + j, make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
            }
        }
        if (contributors > 1 && tid == 0) p.counters[s.tile] = 0;
    }
    if (contributors == 1) release_accumulator();
    if (tid == 0) { TL(5, seg_idx * 8 + 4); }
    bool send = finished;
    if (p.gated) {
        // the second of the pair's two tiles to be finished forms the product (the same four warps run through the same
        // barriers whether or not this block finished anything)
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (tid == 0) {
            int second = 0;
            if (finished && (eok || contributors > 1)) second = atomicAdd(p.gate_counters + gate_pair, 1) == 1 ? 1 : 0;
            __threadfence();
            *c.last_flag = second;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        send = *c.last_flag != 0;
        if (send) {
            OutView og = ov;
            og.out = p.outv[0];
            og.bias = nullptr;
#pragma unroll
            for (int cc = 0; cc < NB / 16; ++cc) {
                const int col0 = cc * 16;
                const float4 *g0 = reinterpret_cast<const float4 *>(p.gate + ((int64_t)(gate_pair * 2) * BN + quad * 32 + lane) * NB + col0);
                const float4 *g1 = g0 + (int64_t)BN * NB / 4;
                float v[16];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 x = __ldcg(g0 + j), y = __ldcg(g1 + j);
                    v[4 * j] = x.x * y.x; v[4 * j + 1] = x.y * y.y; v[4 * j + 2] = x.z * y.z; v[4 * j + 3] = x.w * y.w;
                }
                if (TTB_COL_OK) finish_and_store_t<TTB_ACT_NONE>(p, og, v, row0, col0, n, stage);
            }
            if (tid == 0) p.gate_counters[gate_pair] = 0;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");   // (last_flag is reused below)
    }
    if (tid == 0) { TL(5, seg_idx * 8 + 5); }
    if (done_counter) {
        // a later stage of this launch reads this stage's output: count the tile once it is stored
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (tid == 0 && send && (eok || contributors > 1)) atomicAdd(done_counter, 1);
    }
    if (gathered) {
        // one decision for the four warps, so that all of them take part in gather_send's barriers
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (tid == 0) *c.last_flag = (send && *c.abort_flag == 0) ? 1 : 0;
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        if (*c.last_flag) gather_send<NB>(p, stage, row0, tr.nt, tid, kEpiThreads);   // ends with a barrier: the slab is free again
    }
    if (tid == 0) { TL(6, seg_idx); }
    return eok;
#undef TTB_COL_OK
}

template <int FMT, int S, int NB>
__global__ void __launch_bounds__(kThreads, 1) matmul_decode_tmem_kernel(const __grid_constant__ Sequence<S> q) {
    using L = Layout<FMT, NB>;
    constexpr int kRing = L::kRing;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + L::bars;
    constexpr int kWRing = L::kWRing;
    auto full_b = [&](int s) { return bar0 + 8u * s; };                   // the group's activations have landed
    auto full_a = [&](int s) { return bar0 + 8u * (kRing + s); };         // the group's weights are expanded in tensor memory
    auto empty = [&](int s) { return bar0 + 8u * (2 * kRing + (s >> 1)); };   // the MMAs of the pair of groups {s & ~1, s | 1} are complete: both slots are free
    const uint32_t acc_full0 = bar0 + 8u * (3 * kRing), acc_empty0 = acc_full0 + 16u;
    // the ring of packed tiles (slot = group number modulo kWRing): landed / read out of shared memory (the slot can take
    // the next copy while the expanded weights still wait in tensor memory for their MMAs)
    auto full_w = [&](int s) { return acc_empty0 + 16u + 8u * s; };
    auto w_empty = [&](int s) { return acc_empty0 + 16u + 8u * (kWRing + s); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::misc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::misc + 4);
    volatile int *last_flag = reinterpret_cast<volatile int *>(smem + L::misc + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int block = (int)blockIdx.x;
    const DecodeArgs &p0 = q.st[0];
    // (the waits inside the block outlast the wait for other GPUs that some stage of the launch may sit in)
    bool waits_for_peers = false;
#pragma unroll
    for (int s = 0; s < S; ++s) waits_for_peers = waits_for_peers || (s < q.n && q.st[s].wait_arrived != nullptr);
    const long long lim = p0.wait_limit > 0 ? 2 * p0.wait_limit + 1000000LL : waits_for_peers ? 25000000000LL : 2000000000LL;
    int *const status = p0.status;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kRing; ++s) {
            mbar_init(full_b(s), 1);      // the activation producer, with its byte count
            mbar_init(full_a(s), 4);      // the four expand warps of the group's team
            if ((s & 1) == 0) mbar_init(empty(s), 1);   // the commit of the issuer that owns the pair
        }
        for (int s = 0; s < kWRing; ++s) {
            mbar_init(full_w(s), 1);      // the weight producer, with its byte count
            mbar_init(w_empty(s), 4);     // the four expand warps of the group's team
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(acc_full0 + 8u * s, 2);
            mbar_init(acc_empty0 + 8u * s, 4);
        }
        *abort_flag = 0;
        *last_flag = 0;
        fence_mbar_init();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(sbase + L::misc, L::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;
    // The next kernel on the stream may start while this grid drains; before grid_dep_wait() a role reads nothing but
    // packed weights.
    grid_dep_launch();

    if (warp == kProducerWarp) {
        // ---------------- packed weight tiles -> shared-memory ring, across segment and stage borders ----------------
        // (the whole warp walks the work list, one elected lane issues: see the MMA issuers)
        {
            const bool leader = elect_one();
            const uint64_t policy = l2_policy_evict_first();
            int gs = 0, tlg = 0;
            (void)tlg;
            uint32_t ph = 0;
            WorkIter<S> it;
            it.start(q, block);
            Seg s;
            while (ok && it.next(q, block, s)) {
                const DecodeArgs &p = q.st[S == 1 ? 0 : it.si];
                const TileRef tr = tile_ref(p, s.tile);
                const void *map = &q.maps[S == 1 ? 0 : it.si].m[tr.prob];
                for (int i0 = 0; i0 < s.nit; i0 += kGroup) {
                    if (!__all_sync(0xffffffffu, mbar_wait(w_empty(gs), ph ^ 1, abort_flag, status, 11, lim))) { ok = false; break; }
                    if (leader) {
                        TL(0, tlg);
                        // always a whole box of four K blocks: in a short last group the surplus lands in the group's unused
                        // stages (rows beyond the weight read as zeros), and the byte count the barrier expects stays the same
                        mbar_arrive_expect_tx(full_w(gs), kGroup * L::kStageBytes);
                        tma_load_3d(sbase + L::pk + gs * kGroup * L::kStageBytes, map, 0, tr.nt * 4, s.kb0 + i0, full_w(gs), policy);
                    }
                    ++tlg;
                    if (++gs == kWRing) { gs = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == kLoaderWarp) {
        // ---------------- activations -> shared memory, one tensor-map copy per group ----------------
        {
            const bool leader = elect_one();
            grid_dep_wait();   // the activations are earlier kernels' output
            // What the gather points this launch waits for had been told to expect before the launch (the totals are only
            // brought up to date by the last block to finish); stages of this launch that gather into a point add their share.
            unsigned e0[S];
#pragma unroll
            for (int s = 0; s < S; ++s) e0[s] = (s < q.n && q.st[s].wait_arrived) ? *reinterpret_cast<const volatile unsigned *>(q.st[s].wait_expected) : 0u;
            int gs = 0, tlg = 0, ready_stage = -1;
            (void)tlg;
            uint32_t ph = 0;
            WorkIter<S> it;
            it.start(q, block);
            Seg s;
            while (ok && it.next(q, block, s)) {
                const DecodeArgs &p = q.st[S == 1 ? 0 : it.si];
                if (it.si != ready_stage) {
                    // first segment of a stage: hold the copies until the stage's activation is complete
                    ready_stage = it.si;
                    bool waited = false, good = true;
                    if (p.wait_arrived) {
                        unsigned target = 0;
#pragma unroll
                        for (int j = 0; j < S; ++j) {
                            if (j == it.si) target += e0[j];
                            if (j < it.si && q.st[j].ranks > 1 && q.st[j].expected == p.wait_expected) target += q.st[j].launch_arrivals;
                        }
                        if (leader) good = peer_wait_for(p, target, abort_flag, 6);   // (one lane polls)
                        waited = true;
                    }
                    if (S > 1 && p.depends_on >= 0) {
                        if (leader && good) good = count_wait(q.sync + 1 + p.depends_on, q.st[p.depends_on].sk_tiles / (q.st[p.depends_on].gated ? 2 : 1), p, abort_flag, 8);
                        waited = true;
                    }
                    if (waited) {
                        if (!__all_sync(0xffffffffu, good)) { ok = false; break; }
                        if (leader) fence_proxy_async_global();   // what was stored before the signal is read by the copy unit next
                    }
                    if (leader) { TL(8, it.si); }
                }
                const int rchunk = s.tile / p.tstart[p.nprob];
                const void *amap = &q.amap[S == 1 ? 0 : it.si].m;
                for (int i0 = 0; i0 < s.nit; i0 += kGroup) {
                    if ((gs & 1) == 0 && !__all_sync(0xffffffffu, mbar_wait(empty(gs), ph ^ 1, abort_flag, status, 17, lim))) { ok = false; break; }
                    if (leader) {
                        TL(4, tlg);
                        mbar_arrive_expect_tx(full_b(gs), kGroup * L::kBStageBytes);
                        // one copy per tile row of the block: [tile row][K block][16-column half][32 rows][16 values]
#pragma unroll
                        for (int t = 0; t < NB / 32; ++t) {
                            const uint32_t dst = sbase + L::b + gs * kGroup * L::kBStageBytes + t * kGroup * L::kBRowStage;
                            if (p.a_row_major)
                                tma_load_3d_plain(dst, amap, 0, rchunk * NB + t * 32, (s.kb0 + i0) * 2, full_b(gs));
                            else
                                tma_load_5d(dst, amap, 0, 0, 0, 0, (rchunk * (NB / 32) + t) * p.Kt + s.kb0 + i0, full_b(gs));
                        }
                    }
                    ++tlg;
                    if (++gs == kRing) { gs = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == kMmaWarp || warp == kMmaWarp + 1) {
        // ---------------- MMA issuers: A from tensor memory, B (activations) from shared memory ----------------
        // Issuer h takes the pairs of groups (numbered over the block's whole work) whose pair number is h modulo 2 and
        // accumulates them in accumulator h.
        // The whole warp walks the work list (so that addresses and descriptors stay warp-uniform values); one elected lane
        // issues.
        {
            const bool leader = elect_one();
            const int h = warp - kMmaWarp;
            constexpr uint32_t idesc = instr_desc_bf16_f32(BN, 32, /*a_mn_major=*/false, /*b_mn_major=*/false);   // one MMA per tile row of the block
            const uint64_t b_desc0 = smem_desc_sw32(sbase + L::b, kB_SBO);
            const uint32_t b_lo0 = (uint32_t)b_desc0, b_hi = (uint32_t)(b_desc0 >> 32);
            const uint32_t a_col0 = tmem_base + (uint32_t)L::kACol0;
            auto mk = [](uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; };
            int gs = 0, seg_idx = 0, G = 0;
            uint32_t ph = 0;
            WorkIter<S> it;
            it.start(q, block);
            Seg s;
            for (; ok && it.next(q, block, s); ++seg_idx) {
                const int buf = seg_idx % L::kSets;
                // (every decision the warp takes is taken by all its lanes together)
                if (!__all_sync(0xffffffffu, mbar_wait(acc_empty0 + 8u * buf, (uint32_t)(((seg_idx / L::kSets) & 1) ^ 1), abort_flag, status, 16, lim))) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)((buf * L::kAccs + h) * NB);
                bool fresh = true;   // this issuer's accumulator holds nothing of this segment yet
                for (int i0 = 0; i0 < s.nit; i0 += kGroup) {
                    if (((G >> 1) & 1) == h) {   // (G: the group's number over the block's whole work)
                        const int r = min(kGroup, s.nit - i0);
                        if (h == 0 && leader) { TL(1, G); }
                        if (!__all_sync(0xffffffffu, mbar_wait(full_a(gs), ph, abort_flag, status, 12, lim) && mbar_wait(full_b(gs), ph, abort_flag, status, 18, lim))) { ok = false; break; }
                        if (h == 0 && leader) { TL(2, G); }
                        tc_fence_after_sync();
                        const uint32_t a_col = a_col0 + (uint32_t)(gs * kGroup * kAColsPerStage);
                        const uint32_t b_lo = b_lo0 + (uint32_t)gs * ((kGroup * L::kBStageBytes) >> 4);
#pragma unroll
                        for (int j = 0; j < kGroup; ++j) {
#ifdef TTB_KO_MMA
                            if (false) {
#else
                            if (j < r) {
#endif
                                if (leader) {
                                    // (the activations of a tile row are a K-major operand of 32 rows; its results are 32 columns of the accumulator)
#pragma unroll
                                    for (int t = 0; t < NB / 32; ++t) {
                                        const uint32_t bt = b_lo + (uint32_t)((t * kGroup * L::kBRowStage + j * L::kBRowStage) >> 4);
                                        mma_bf16_ts(d_tmem + (uint32_t)(t * 32), a_col + (uint32_t)(j * kAColsPerStage), mk(bt, b_hi), idesc, !(fresh && j == 0));
                                        mma_bf16_ts(d_tmem + (uint32_t)(t * 32), a_col + (uint32_t)(j * kAColsPerStage + 8), mk(bt + (uint32_t)((L::kBRowStage / 2) >> 4), b_hi), idesc, true);
                                    }
                                }
                            }
                        }
                        fresh = false;
                        if ((gs & 1) && leader) mma_commit(empty(gs));   // second group of the pair: one commit frees both slots
                        if (h == 0 && leader) { TL(3, G); }
                    }
                    ++G;
                    if (++gs == kRing) { gs = 0; ph ^= 1; }
                }
                // (an issuer that had no group in this segment still commits: its arrival is part of the barrier's count)
                if (ok && leader) mma_commit(acc_full0 + 8u * buf);
            }
            // An odd number of groups leaves the last pair's commit unsent: nothing waits for it any more.
        }
    } else if (warp >= kEpiWarp0) {
        // ---------------- epilogue warps ----------------
        grid_dep_wait();   // the epilogues touch scratch and outputs
        const EpiCtx ectx = {smem, tmem_base, acc_full0, acc_empty0, abort_flag, last_flag, lim};
        int seg_idx = 0, g0 = 0;
        WorkIter<S> it;
        it.start(q, block);
        Seg s;
        for (; it.next(q, block, s); ++seg_idx) {
            const DecodeArgs &p = q.st[S == 1 ? 0 : it.si];
            ok = epilogue<FMT, NB>(p, ectx, s, seg_idx, g0, ok, (S > 1 && p.count_done) ? q.sync + 1 + it.si : nullptr);
            g0 += (s.nit + kGroup - 1) / kGroup;
        }
    } else {
        // ---------------- expand warps: packed codes -> bf16 in tensor memory ----------------
        const int team = warp >> 2, quad = warp & 3;
        // ldmatrix row addresses: lanes 0-15 give the rows of the left face, 16-31 of the right face
        const uint32_t ld_off = 64u + (uint32_t)(lane >> 4) * 256u + (uint32_t)(lane & 15) * 16u;
        // bfloat4_b: a 16-byte row of the transposing load is a pair of K rows of one face (8 bytes = 16 nibbles each). Lanes
        // 0-15 give the rows of the left faces (0 and 2), lanes 16-31 of the right faces; row r of the 16 is K row pair
        // sigma(r) of the upper (sigma < 8) or lower face, with sigma chosen such that the four rows a lane receives
        // (4q .. 4q+3, q = lane % 4) are K rows 4q..4q+3 of the upper and of the lower face - the same K rows a lane holds
        // for bfloat8_b, so the scale table and the TMEM columns are the same.
        const int r16 = lane & 15;
        const int sigma = ((r16 >> 1) & 1) * 8 + (r16 >> 2) * 2 + (r16 & 1);   // 0,1,8,9, 2,3,10,11, 4,5,12,13, 6,7,14,15
        const uint32_t ld_off4 = 64u + (uint32_t)(lane >> 4) * 128u + (uint32_t)(sigma >> 3) * 256u + (uint32_t)(sigma & 7) * 16u;
        const int sh0 = 2 * (lane & 3);  // within a face's 8 scale pairs: this lane's K rows are 4*(lane%4) .. +3
        const uint32_t st_lane = (uint32_t)(quad * 32) << 16;
        const uint32_t pk_quad = sbase + L::pk + quad * L::kTile;
        const uint32_t a_col_q = tmem_base + st_lane + (uint32_t)L::kACol0;
        // the block's groups are numbered across segments and stages; team t takes groups t, t + 3, ...
        WorkIter<S> it;
        it.start(q, block);
        Seg cur = {0, 0, 0, 1, 0, 0};
        int cur_g0 = 0, cur_ng = 0;
        auto locate = [&](int G) {   // advances `cur` to the segment that holds group G; false once the block's work ends
            while (G >= cur_g0 + cur_ng) {
                cur_g0 += cur_ng;
                if (!it.next(q, block, cur)) {
                    cur_ng = 0;
                    return false;
                }
                cur_ng = (cur.nit + kGroup - 1) / kGroup;
            }
            return true;
        };
        int G = team;
        int gs = G % kRing, ws = G % kWRing;   // (ws: the slot in the ring of packed tiles)
        uint32_t phs = (uint32_t)(G / kRing) & 1u, wphs = (uint32_t)(G / kWRing) & 1u;
        while (locate(G)) {
            const int r = min(kGroup, cur.nit - (G - cur_g0) * kGroup);
            int good = 1;
            if (lane == 0 && quad == 0) { TL(7, G); }
            // the packed tiles have landed, and the MMAs that read this slot's place in tensor memory a ring pass ago are complete
            good = mbar_wait(full_w(ws), wphs, abort_flag, status, 14, lim) && mbar_wait(empty(gs), phs ^ 1u, abort_flag, status, 19, lim);
            if (!__all_sync(0xffffffffu, good)) { ok = false; break; }
            if (lane == 0 && quad == 0) { TL(9, G); }
            tc_fence_after_sync();
            uint32_t tile = pk_quad + (uint32_t)(ws * kGroup * L::kStageBytes);
            uint32_t a_col = a_col_q + (uint32_t)(gs * kGroup * kAColsPerStage);
#ifdef TTB_KO_EXPAND
            if (false)
#endif
#pragma unroll 1
            for (int j = 0; j < r; j += 2) {
                // row scales: lane l holds the powers of two of exponent bytes 2l and 2l+1 of the tile's 64
                const bool two = j + 1 < r;
                uint32_t e2, e3 = 0u;
                asm volatile("ld.shared.u16 %0, [%1];" : "=r"(e2) : "r"(tile + 2u * lane));
                if (two) asm volatile("ld.shared.u16 %0, [%1];" : "=r"(e3) : "r"(tile + (uint32_t)L::kStageBytes + 2u * lane));
                const uint32_t eh = __byte_perm(e2, 0u, 0x4140u), eh1 = __byte_perm(e3, 0u, 0x4140u);   // [e0, 0, e1, 0]
                const bool big = __any_sync(0xffffffffu, ((eh | eh1) & 0x00800080u) != 0u);
                if (two && !big) {
                    if (FMT == TTB_BFLOAT8_B)
                        expand_pair(tile, tile + L::kStageBytes, a_col, a_col + kAColsPerStage, ld_off, eh, eh1, sh0);
                    else
                        expand_pair4(tile, tile + L::kStageBytes, a_col, a_col + kAColsPerStage, ld_off4, eh, eh1, sh0);
                } else {
                    // a lone last tile, or an exponent above 127 somewhere (a row maximum of 2 or more): one tile at a time
                    for (int t = 0; t < (two ? 2 : 1); ++t) {
                        const uint32_t e = t ? eh1 : eh, tl = tile + (uint32_t)(t * L::kStageBytes), ac = a_col + (uint32_t)(t * kAColsPerStage);
                        const bool b1 = __any_sync(0xffffffffu, (e & 0x00800080u) != 0u);
                        if (FMT == TTB_BFLOAT8_B) {
                            if (b1)
                                expand_tile_big(tl, ac, ld_off, e, sh0);
                            else
                                expand_tile<false>(tl, ac, ld_off, e, sh0);
                        } else {
                            if (b1)
                                expand_tile4_big(tl, ac, ld_off4, e, sh0);
                            else
                                expand_tile4<false>(tl, ac, ld_off4, e, sh0);
                        }
                    }
                }
                tile += 2 * L::kStageBytes;
                a_col += 2 * kAColsPerStage;
            }
            if (lane == 0 && quad == 0) { TL(10, G); }
            tmem_st_wait();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(full_a(gs));
                mbar_arrive(w_empty(ws));
            }
            if (lane == 0 && quad == 0) { TL(11, G); }
            G += kTeams;
            gs += kTeams;
            if (gs >= kRing) { gs -= kRing; phs ^= 1u; }
            ws += kTeams;
            if (ws >= kWRing) { ws -= kWRing; wphs ^= 1u; }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // A wait ran out: give copies and MMAs still in flight a bounded time to land before the block's shared memory
        // and tensor memory are released.
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, L::kTmemCols);
    }
    // The last block to finish brings the gather points' expected totals up to date (nothing in this launch reads them
    // after its start) and leaves the launch's bookkeeping counters zero.
    if (threadIdx.x == 0) {
        grid_dep_wait();   // (a block without work gets here early: the counters may still be the previous launch's)
        bool last = gridDim.x == 1;
        if (q.sync && gridDim.x > 1) {
            __threadfence();
            last = atomicAdd(q.sync, 1) == (int)gridDim.x - 1;
        } else if (!q.sync) {
            last = block == 0;   // a single stage without scratch: no stage of this launch waits on a point it fills
        }
        if (last) {
            for (int s = 0; s < q.n; ++s) {
                if (q.st[s].ranks > 1) *q.st[s].expected = *q.st[s].expected + q.st[s].launch_arrivals;
                if (q.sync) q.sync[1 + s] = 0;
            }
            if (q.sync) q.sync[0] = 0;
        }
    }
}

template <int FMT, int S, int NB>
int32_t launch_seq(const Sequence<S> &q, bool overlap, cudaStream_t stream) {
    constexpr int smem_bytes = Layout<FMT, NB>::total + 1024;
    static_assert(smem_bytes <= 232448, "shared memory budget");
    static bool configured[64] = {};
    int dev = 0;
    TTB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        TTB_CUDA_TRY(cudaFuncSetAttribute(matmul_decode_tmem_kernel<FMT, S, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)q.grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    TTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, matmul_decode_tmem_kernel<FMT, S, NB>, q));
    TTB_LAUNCH_CHECK("matmul_decode_tmem");
    return TTB_OK;
}

template <int S>
int32_t build_and_launch(const DecodeArgs *stages, int n, int fmt, int nb, int *sync, bool overlap, cudaStream_t stream) {
    static Sequence<S> q;   // (large: kept out of the stack; one host thread per process drives the library)
    q.n = n;
    q.sync = sync;
    q.grid = 1;
    for (int s = 0; s < n; ++s) {
        q.st[s] = stages[s];
        if (stages[s].sk_grid > q.grid) q.grid = stages[s].sk_grid;
        if (int32_t rc = make_weight_maps(stages[s], fmt, q.maps[s], kGroup)) return rc;
        if (int32_t rc = make_act_map(stages[s], (int64_t)(stages[s].sk_tiles / stages[s].tstart[stages[s].nprob]) * nb, q.amap[s], kGroup)) return rc;
    }
    if constexpr (S == 1) {
        if (nb == 64) {
            if (fmt == TTB_BFLOAT8_B) return launch_seq<TTB_BFLOAT8_B, S, 64>(q, overlap, stream);
            return launch_seq<TTB_BFLOAT4_B, S, 64>(q, overlap, stream);
        }
    }
    if (fmt == TTB_BFLOAT8_B) return launch_seq<TTB_BFLOAT8_B, S, 32>(q, overlap, stream);
    return launch_seq<TTB_BFLOAT4_B, S, 32>(q, overlap, stream);
}

}  // namespace

#ifdef TTB_TIMELINE
extern "C" int32_t ttb_debug_timeline(void *host) {
    TTB_CUDA_TRY(cudaMemcpyFromSymbol(host, g_tl, sizeof(g_tl)));
    return TTB_OK;
}

#endif

// `stages`: what launch_matmul_decode_multi prepared for each stage (blocks of `nb` rows, one weight format for the launch);
// `sync`: the launch's bookkeeping counters in the zeroed head of the workspace, or null for a single stage without scratch.
int32_t launch_decode_tmem(const DecodeArgs *stages, int n, int fmt, int nb, int *sync, bool overlap, cudaStream_t stream) {
    if (n < 1 || n > kMaxSequenceStages) return fail(TTB_E_INVALID, "a launch holds 1..%d stages", kMaxSequenceStages);
    if (nb != 32 && nb != 64) return fail(TTB_E_INVALID, "the tensor-memory decode kernel takes blocks of 32 or 64 rows");
    if (n == 1) return build_and_launch<1>(stages, n, fmt, nb, sync, overlap, stream);
    if (nb != 32) return fail(TTB_E_UNSUPPORTED, "several stages in one launch need one tile row per block");
    return build_and_launch<kMaxSequenceStages>(stages, n, fmt, nb, sync, overlap, stream);
}

}  // namespace ttb
