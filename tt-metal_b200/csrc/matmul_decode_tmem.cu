// Weight-streaming decode matmul for bfloat8_b weights with the weight operand fed to the tensor cores through
// tensor memory instead of shared memory.
//
// out[rows, N] = act(a[rows, K] x W[K, N] + bias), rows in {32, 64, 128} per block, "swap-AB" as in
// matmul_decode_stream.cu: the MMA's M dimension (128 TMEM lanes) runs over weight columns, its N dimension over the
// activation rows.
//
// Why tensor memory: expanded to bf16 a weight is two bytes, and writing it to shared memory and having the MMA
// fetch it back costs four bytes of shared-memory traffic per weight - more than the shared-memory pipe can move at
// the rate HBM delivers the one packed byte. Here the packed tile goes through shared memory once (bulk copy in,
// ldmatrix out) and the bf16 values go registers -> tensor memory -> MMA:
//   * ldmatrix.m16n16.trans.b8 reads a 16x16 face of 8-bit codes transposed, so that a lane holds four consecutive
//     K values of one weight column - the order the MMA's A operand wants (TMEM lane = column n, TMEM column = K pair);
//   * the codes become bf16 with one byte-permute, one mask and one packed multiply per pair (subnormal trick:
//     (sign << 15) | mantissa is the weight divided by 2^E), the per-row powers of two coming from a warp-wide
//     table of the tile's 64 exponents (one pair per lane, fetched by shuffle);
//   * tcgen05.st.16x256b has exactly the fragment layout ldmatrix produced, so the expanded registers go to tensor
//     memory without any shuffle; tcgen05.mma then takes A from tensor memory and the activations (B) from shared memory.
// A warp can only write the 32 TMEM lanes of its quadrant (warp % 4), i.e. one tile column of the 128-wide block, so
// the twelve expand warps form three teams of four (one warp per quadrant): team t expands every third group of three
// K-blocks, all three stages in one turn. One mbarrier per group keeps the producer thread, the MMA-issuing thread and
// the expand warps to one wait / commit / arrival per three stages.
// Every mbarrier wait is bounded; a wait that runs out raises a status word instead of hanging.
#include "decode_common.cuh"

namespace ttb {
namespace {

using namespace ptx;

constexpr int BN = 128;  // weight columns per block (MMA M, TMEM lanes)
constexpr int BK = 32;   // K per stage: one row of four packed tiles
constexpr int kSets = 3;                       // expand-warp sets = stages per group
constexpr int kExpandWarps = 4 * kSets;        // warps 0..11; quadrant = warp % 4, set = warp / 4
constexpr int kProducerWarp = 12, kMmaWarp = 13;
constexpr int kThreads = 32 * 14;
constexpr int kEpilogueThreads = 32 * kExpandWarps;
constexpr int kTile = kBfp8TileBytes;
constexpr int kStageBytes = 4 * kTile;         // 4352
constexpr int kPkGroups = 8;                   // packed ring: 24 stages = 102 KiB in flight
constexpr int kAGroups = 4;                    // TMEM A ring: 12 stages x 16 columns
constexpr int kAColsPerStage = BK / 2;
constexpr uint32_t kB_LBO = 128, kB_SBO = 512;  // activations, K-contiguous canonical layout without swizzle

template <int NB>
struct Layout {
    static constexpr int kBStageBytes = NB * BK * 2;
    static constexpr int pk = 0;
    static constexpr int b = pk + kPkGroups * kSets * kStageBytes;
    static constexpr int bars = b + kAGroups * kSets * kBStageBytes;
    static constexpr int nbars = 2 * kPkGroups + 2 * kAGroups + 1;
    static constexpr int misc = bars + 8 * nbars;
    static constexpr int total = misc + 16;
    static constexpr int kAccCols = 2 * NB;                        // one accumulator per K step of a stage
    static constexpr int kACol0 = kAccCols;                        // the A ring follows the accumulators
    static constexpr int kTmemColsUsed = kAccCols + kAGroups * kSets * kAColsPerStage;
    static constexpr int kTmemCols = kTmemColsUsed <= 256 ? 256 : 512;
};

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

// Four codes (consecutive K of one column) -> two packed bf16 pairs, each multiplied by its pair of row scales.
__device__ __forceinline__ void expand4(uint32_t codes, uint32_t s01, uint32_t s23, uint32_t &o01, uint32_t &o23) {
    uint32_t x01 = __byte_perm(codes, 0u, 0x1100u) & 0x807f807fu;
    uint32_t x23 = __byte_perm(codes, 0u, 0x3322u) & 0x807f807fu;
    __nv_bfloat162 v01 = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&x01), *reinterpret_cast<__nv_bfloat162 *>(&s01));
    __nv_bfloat162 v23 = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&x23), *reinterpret_cast<__nv_bfloat162 *>(&s23));
    o01 = *reinterpret_cast<uint32_t *>(&v01);
    o23 = *reinterpret_cast<uint32_t *>(&v23);
}
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
    __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&a), *reinterpret_cast<__nv_bfloat162 *>(&b));
    return *reinterpret_cast<uint32_t *>(&v);
}

template <int NB>
__global__ void __launch_bounds__(kThreads, 1) matmul_decode_tmem_kernel(const DecodeArgs p) {
    using L = Layout<NB>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + L::bars;
    auto full_pk = [&](int s) { return bar0 + 8u * s; };
    auto empty_pk = [&](int s) { return bar0 + 8u * (kPkGroups + s); };
    auto full_a = [&](int s) { return bar0 + 8u * (2 * kPkGroups + s); };
    auto empty_a = [&](int s) { return bar0 + 8u * (2 * kPkGroups + kAGroups + s); };
    const uint32_t accum_bar = bar0 + 8u * (2 * kPkGroups + 2 * kAGroups);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::misc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::misc + 4);
    volatile int *last_flag = reinterpret_cast<volatile int *>(smem + L::misc + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntile = blockIdx.x, split = blockIdx.y, rchunk = blockIdx.z;
    const int kb0 = split * p.kb_per_split;
    const int nit = min(p.nkb, kb0 + p.kb_per_split) - kb0;
    const int ngroups = (nit + kSets - 1) / kSets;
    const int64_t row0 = (int64_t)rchunk * NB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPkGroups; ++s) {
            mbar_init(full_pk(s), 1);
            mbar_init(empty_pk(s), 4);
        }
        for (int s = 0; s < kAGroups; ++s) {
            mbar_init(full_a(s), 4);
            mbar_init(empty_a(s), 1);
        }
        mbar_init(accum_bar, 1);
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
    // As in the shared-memory kernel: the next kernel may start while this grid drains, and only the packed weights are
    // read before grid_dep_wait().
    grid_dep_launch();

    if (warp == kProducerWarp) {
        // ---------------- producer: packed weight tiles -> shared-memory ring, three stages per barrier ----------------
        if (lane == 0) {
            const uint64_t policy = l2_policy_evict_first();
            const uint8_t *src = p.w + ((int64_t)kb0 * p.Nt + (int64_t)ntile * 4) * kTile;
            const int64_t src_step = (int64_t)p.Nt * kTile;
            int gs = 0;
            uint32_t ph = 0;
            for (int g = 0; g < ngroups; ++g) {
                const int r = min(kSets, nit - g * kSets);
                if (!mbar_wait(empty_pk(gs), ph ^ 1, abort_flag, p.status, 11)) { ok = false; break; }
                mbar_arrive_expect_tx(full_pk(gs), r * kStageBytes);
                for (int j = 0; j < r; ++j) {
                    bulk_g2s(sbase + L::pk + (gs * kSets + j) * kStageBytes, src, kStageBytes, full_pk(gs), policy);
                    src += src_step;
                }
                if (++gs == kPkGroups) { gs = 0; ph ^= 1; }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer: A from tensor memory, B (activations) from shared memory ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16_f32(BN, NB, /*a_mn_major=*/false, /*b_mn_major=*/false);
            const uint64_t b_desc0 = smem_desc_noswizzle(sbase + L::b, kB_LBO, kB_SBO);
            const uint32_t b_lo0 = (uint32_t)b_desc0, b_hi = (uint32_t)(b_desc0 >> 32);
            auto mk = [](uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; };
            int ga = 0;
            uint32_t ph = 0;
            for (int g = 0; g < ngroups; ++g) {
                const int r = min(kSets, nit - g * kSets);
                if (!mbar_wait(full_a(ga), ph, abort_flag, p.status, 12)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t a_col = tmem_base + (uint32_t)(L::kACol0 + ga * kSets * kAColsPerStage);
                const uint32_t b_lo = b_lo0 + (uint32_t)ga * ((kSets * L::kBStageBytes) >> 4);
#pragma unroll
                for (int j = 0; j < kSets; ++j) {
                    if (j < r) {
#pragma unroll
                        for (int k16 = 0; k16 < BK / 16; ++k16)
                            mma_bf16_ts(tmem_base + (uint32_t)(k16 * NB), a_col + (uint32_t)(j * kAColsPerStage + k16 * 8),
                                        mk(b_lo + ((j * L::kBStageBytes + k16 * 2 * kB_LBO) >> 4), b_hi), idesc, j > 0 || g > 0);
                    }
                }
                mma_commit(empty_a(ga));
                if (++ga == kAGroups) { ga = 0; ph ^= 1; }
            }
            if (ok) mma_commit(accum_bar);
        }
    } else {
        // ---------------- expand warps: packed codes -> bf16 in tensor memory; activations -> shared memory ----------------
        // Team warp / 4 (four warps, one per TMEM lane quadrant = tile column) takes every third group and expands all
        // of its stages in one turn, so the per-turn costs (barrier polls, fences, arrivals) are paid once per three stages.
        const int team = warp >> 2, quad = warp & 3;
        constexpr int kActChunks = NB / 32;  // 16-byte activation chunks per lane per stage (NB rows x 4 chunks over 4 warps)
        uint4 act_regs[kSets][kActChunks];
        // per-lane source pointers of this lane's chunks at K-block 0 of the block's K range; K-block it is it * step further
        const uint16_t *act_src[kActChunks];
#pragma unroll
        for (int q = 0; q < kActChunks; ++q) {
            const int c = q * 128 + quad * 32 + lane;
            act_src[q] = p.a + act_chunk_base(p, row0 + c % NB, c / NB) + (int64_t)kb0 * act_chunk_step(p);
        }
        const int act_step = act_chunk_step(p);
        grid_dep_wait();
        auto load_act = [&](int g) {
#pragma unroll
            for (int j = 0; j < kSets; ++j) {
                const int it = g * kSets + j;
                if (it < nit) {
#pragma unroll
                    for (int q = 0; q < kActChunks; ++q)
                        act_regs[j][q] = __ldg(reinterpret_cast<const uint4 *>(act_src[q] + (int64_t)it * act_step));
                }
            }
        };
        if (team < ngroups) load_act(team);
        // ldmatrix row addresses: lanes 0-15 give the rows of the left face, 16-31 of the right face
        const uint32_t ld_off = 64u + (uint32_t)(lane >> 4) * 256u + (uint32_t)(lane & 15) * 16u;
        const int sh0 = 2 * (lane & 3);  // within a face's 8 scale pairs: this lane's K rows are 4*(lane%4) .. +3
        const uint32_t st_lane = (uint32_t)(quad * 32) << 16;
        for (int g = team; g < ngroups; g += kSets) {
            const int r = min(kSets, nit - g * kSets);
            const int gs = g % kPkGroups, ga = g % kAGroups;
            const uint32_t phs = (g / kPkGroups) & 1, pha = (g / kAGroups) & 1;
            int good = 1;
            if (lane == 0)
                good = mbar_wait(empty_a(ga), pha ^ 1, abort_flag, p.status, 13) && mbar_wait(full_pk(gs), phs, abort_flag, p.status, 14);
            good = __shfl_sync(0xffffffffu, good, 0);
            if (!good) { ok = false; break; }
#pragma unroll
            for (int j = 0; j < kSets; ++j) {
                if (j < r) {
                    const uint32_t tile = sbase + L::pk + (gs * kSets + j) * kStageBytes + quad * kTile;
                    // row scales: lane l holds the powers of two of exponent bytes 2l and 2l+1 of the tile's 64
                    const uint32_t e2 = *reinterpret_cast<const uint16_t *>(smem + (tile - sbase) + 2 * lane);
                    const uint32_t eh = __byte_perm(e2, 0u, 0x4140u);                 // [e0, 0, e1, 0]
                    const uint32_t my_scale = (__vminu2(eh, 0x007f007fu) + 0x007f007fu) << 7;   // 2^min(E, 127) per half
                    const bool big = __any_sync(0xffffffffu, ((eh | (eh >> 16)) & 0x80u) != 0u);
                    uint32_t top[4], bot[4];
                    ldmatrix_x2_trans_b8(tile + ld_off, top);         // faces 0 (left) and 1 (right): K 0..15
                    ldmatrix_x2_trans_b8(tile + ld_off + 512u, bot);  // faces 2 and 3: K 16..31
                    const uint32_t a_col = tmem_base + st_lane + (uint32_t)(L::kACol0 + (ga * kSets + j) * kAColsPerStage);
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
                        if (big) {
                            // exponents above 127 (row maximum of 2 or more): second factor 2^(E - 127)
                            const uint32_t my_t = __vmaxu2(__vminu2(eh, 0x00fe00feu), 0x007f007fu) << 7;
                            const uint32_t t01 = __shfl_sync(0xffffffffu, my_t, 8 * f + sh0);
                            const uint32_t t23 = __shfl_sync(0xffffffffu, my_t, 8 * f + sh0 + 1);
                            o[0] = mul2(o[0], t01); o[1] = mul2(o[1], t23); o[2] = mul2(o[2], t01); o[3] = mul2(o[3], t23);
                        }
                        // TMEM lanes 32*quad + 16*nh + {lane/4, lane/4 + 8}; columns: stage base + 8*kh + 2*(lane%4) + {0, 1}
                        tmem_st_16x256b(a_col + ((uint32_t)((f & 1) * 16) << 16) + (uint32_t)((f >> 1) * 8), o[0], o[1], o[2], o[3]);
                    }
                    // activations of this K-block (fetched one turn ahead): this warp stores a quarter of the block
                    uint8_t *const bst = smem + L::b + (ga * kSets + j) * L::kBStageBytes;
#pragma unroll
                    for (int q = 0; q < kActChunks; ++q) {
                        const int c = q * 128 + quad * 32 + lane;
                        const int m = c % NB, kc = c / NB;
                        *reinterpret_cast<uint4 *>(bst + (m >> 3) * kB_SBO + kc * kB_LBO + (m & 7) * 16) = act_regs[j][q];
                    }
                }
            }
            tmem_st_wait();
            fence_proxy_async_smem();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(full_a(ga));
            if (lane == 1) mbar_arrive(empty_pk(gs));
            if (g + kSets < ngroups) load_act(g + kSets);
        }
    }

    if (warp < kExpandWarps) {
        // ---------------- epilogue: TMEM lane quadrant warp % 4; the three warps of a quadrant share the columns ----------------
        const int tid = threadIdx.x;
        const int set = warp >> 2, quad = warp & 3;
        grid_dep_wait();
        {
            int good = ok ? 1 : 0;
            if (lane == 0 && good && nit > 0) good = mbar_wait(accum_bar, 0, abort_flag, p.status, 15);
            ok = __shfl_sync(0xffffffffu, good, 0) != 0;
        }
        tc_fence_after_sync();
        const int64_t n = (int64_t)ntile * BN + quad * 32 + lane;
        const int tile_id = rchunk * gridDim.x + ntile;
        if (ok && nit > 0) {
            for (int cc = set; cc < NB / 16; cc += kSets) {
                const int col0 = cc * 16;
                float v[16];
                uint32_t r0[16], r1[16];
                tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)col0, r0);
                tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(NB + col0), r1);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r0[j]) + __uint_as_float(r1[j]);
                if (p.splits == 1) {
                    finish_and_store<NB>(p, v, row0, col0, n);
                } else if (p.ordered) {
                    float4 *dst = reinterpret_cast<float4 *>(
                        p.partial + (((int64_t)tile_id * p.splits + split) * BN + quad * 32 + lane) * NB + col0);
#pragma unroll
                    for (int j = 0; j < 4; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                } else {
                    float *dst = p.accum + ((int64_t)tile_id * BN + quad * 32 + lane) * NB + col0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) red_add_f32x4(dst + 4 * j, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                }
            }
        }
        if (p.splits > 1) {
            // The last block to arrive for this output tile adds all partials in split order and finishes.
            __threadfence();
            asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
            if (tid == 0) *last_flag = (atomicAdd(p.counters + tile_id, 1) == p.splits - 1) ? 1 : 0;
            asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
            if (*last_flag) {
                __threadfence();
                for (int cc = set; cc < NB / 16; cc += kSets) {
                    const int col0 = cc * 16;
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                    if (p.ordered) {
                        // four splits per round: all sixteen loads are issued before the first add, the adds stay in split order
                        for (int sp0 = 0; sp0 < p.splits; sp0 += 4) {
                            float4 x[4][4];
    #pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const int sp = min(sp0 + u, p.splits - 1);
                                const float4 *src = reinterpret_cast<const float4 *>(
                                    p.partial + (((int64_t)tile_id * p.splits + sp) * BN + quad * 32 + lane) * NB + col0);
    #pragma unroll
                                for (int j = 0; j < 4; ++j) x[u][j] = __ldcg(src + j);
                            }
    #pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                if (sp0 + u < p.splits) {
    #pragma unroll
                                    for (int j = 0; j < 4; ++j) {
                                        v[4 * j] += x[u][j].x; v[4 * j + 1] += x[u][j].y; v[4 * j + 2] += x[u][j].z; v[4 * j + 3] += x[u][j].w;
                                    }
                                }
                            }
                        }
                    } else {
                        // the tile's sums are complete: read them and leave zeros behind for the next launch
                        float4 *acc = reinterpret_cast<float4 *>(p.accum + ((int64_t)tile_id * BN + quad * 32 + lane) * NB + col0);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float4 x = __ldcg(acc + j);
                            v[4 * j] = x.x; v[4 * j + 1] = x.y; v[4 * j + 2] = x.z; v[4 * j + 3] = x.w;
                            acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                    }
                    finish_and_store<NB>(p, v, row0, col0, n);
                }
                if (tid == 0) p.counters[tile_id] = 0;  // leave the scratch ready for the next launch
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // A wait ran out: give copies and MMAs still in flight a bounded time to land before the block's
        // shared memory and tensor memory are released.
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) __nanosleep(1000);
        __syncthreads();
    }
    if (warp == kMmaWarp) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, L::kTmemCols);
    }
}

template <int NB>
int32_t launch_one(const DecodeArgs &p, dim3 grid, bool overlap, cudaStream_t stream) {
    constexpr int smem_bytes = Layout<NB>::total + 128;
    static bool configured[64] = {};
    int dev = 0;
    TTB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        TTB_CUDA_TRY(cudaFuncSetAttribute(matmul_decode_tmem_kernel<NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    TTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, matmul_decode_tmem_kernel<NB>, p));
    TTB_LAUNCH_CHECK("matmul_decode_tmem");
    return TTB_OK;
}

}  // namespace

int32_t launch_decode_tmem(const DecodeArgs &p, int nb, dim3 grid, bool overlap, cudaStream_t stream) {
    if (nb == 32) return launch_one<32>(p, grid, overlap, stream);
    if (nb == 64) return launch_one<64>(p, grid, overlap, stream);
    return launch_one<128>(p, grid, overlap, stream);
}

}  // namespace ttb
