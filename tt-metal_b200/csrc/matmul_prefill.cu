// Compute-bound matmul for large row counts (prefill): out[rows, N] = act(a[rows, K] x W[K, N] + bias) with W in
// packed bfloat8_b / bfloat4_b tiles and rows a multiple of 128.
//
// One block owns a [128*R rows] x [128*H columns] output tile (R = H = 2 when the shape allows: 256 x 256, all of tensor
// memory as two fp32 accumulators of 128 lanes x 256 columns; else 256 x 128 or 128 x 128) and walks K in blocks of 32:
//   * the activations are first re-laid once per call (relayout_activations below) into blocks that already have the
//     tensor cores' canonical K-major operand layout, so that the producer can fetch the [128*R x 32] activation
//     block of a K step with one bulk copy; the same warp streams the packed weight tiles of the K step;
//   * the expand warps turn packed codes into bf16 in shared memory in the canonical N-contiguous operand layout
//     (the expansion of matmul_decode_stream.cu, here feeding the MMA's B operand), in teams that take ring groups in turn;
//   * one warp issues tcgen05.mma (M = 128 activation rows, N = 128*H weight columns, K = 16 per instruction, 2*R per
//     K block), accumulating in tensor memory; tcgen05.commit releases operand stages. Producer and issuer run
//     warp-uniform with one elected issuing lane;
//   * eight warps read the accumulators back with tcgen05.ld and apply bias, activation and the bf16 / fp32 store.
// Each expanded weight is reused for 128*R rows, so the expansion cost per flop falls with R; each weight tile is
// expanded once per row block, the packed bytes coming from L2 after their first read. Row blocks vary fastest over the
// grid, and column blocks that would not fill a whole wave of blocks go to a second launch with 128 x 128 blocks.
// Every mbarrier wait is bounded; a wait that runs out raises a status word instead of hanging.
#include <type_traits>

#include "decode_common.cuh"

namespace ttb {
namespace {

using namespace ptx;

constexpr int BMS = 128;  // rows per accumulator (MMA M)
constexpr int BN = 128;   // weight columns per block (MMA N)
constexpr int BK = 32;    // K per stage: one row of four packed tiles
constexpr int kWarps = 12;  // warp 0 producer, warp 4 MMA issuer, warp 8 idle (scheduler 0); the other nine expand
constexpr int kThreads = 32 * kWarps;
constexpr int kExpandWarps = 9;
constexpr int kProducerWarp = 0, kMmaWarp = 4;
// Ring configuration. H = 128-column halves per block (block width 128 * H). With H = 1 stages travel in groups of
// three and the nine expand warps form three teams of three (one stage each); with H = 2 (twice the bytes per stage) in
// groups of two, and eight expand warps form two teams of four (one half of one stage each).
// A team takes every kTeams-th group. Several teams wait on the same ring barriers with different phase parities; a
// parity wait is only right while the waiter is at most one phase behind, which holds as long as no ring has fewer groups
// than there are teams (a team's previous group then already needed the phase before the one it waits for).
template <int H>
struct Cfg {
    static constexpr int kGroup = H == 2 ? 2 : 3;       // stages per barrier group
    static constexpr int kPkGroups = H == 2 ? 2 : 4;    // packed weight ring
    static constexpr int kWGroups = 3;                  // expanded weight ring: stages of H * 8 KiB
    static constexpr int kActGroups = H == 2 ? 3 : 2;   // activation ring: stages of R * 8 KiB
    static constexpr int kTeams = H == 2 ? 2 : 3;       // teams of expand warps
    static constexpr int kMembers = kGroup * H;         // warps per team: one 128-column half of one stage each
    static constexpr int kWStageBytes = H * BN * BK * 2;
    static_assert(kTeams <= kPkGroups && kTeams <= kWGroups, "a ring with fewer groups than teams breaks the parity waits");
    static_assert(kTeams * kMembers <= kExpandWarps, "expand warps");
};
constexpr int kActSubBytes = BMS * BK * 2;       // one 128-row activation sub-block of a K step
constexpr uint32_t kW_LBO = 128, kW_SBO = 512;   // weights (N-contiguous): K-groups adjacent, N-groups 512 B apart
constexpr uint32_t kX_LBO = 128, kX_SBO = 512;   // activations (K-contiguous): K-groups adjacent, row-groups 512 B apart

template <int FMT>
struct Pk {
    static constexpr int kTileBytes = FMT == TTB_BFLOAT8_B ? kBfp8TileBytes : kBfp4TileBytes;
    static constexpr int kRunBytes = 4 * kTileBytes;    // the four tiles of one 128-column half for one K block
};

template <int FMT, int R, int H>
struct Layout {
    using C = Cfg<H>;
    static constexpr int kPkStageBytes = H * Pk<FMT>::kRunBytes;   // the halves of a block are adjacent in the weight
    static constexpr int kActStageBytes = R * kActSubBytes;
    static constexpr int pk = 0;
    static constexpr int w = pk + C::kPkGroups * C::kGroup * kPkStageBytes;
    static constexpr int x = w + C::kWGroups * C::kGroup * C::kWStageBytes;
    static constexpr int bars = x + C::kActGroups * C::kGroup * kActStageBytes;
    // barriers: full_pk, empty_pk [kPkGroups]; full_w, empty_w [kWGroups]; full_x, empty_x [kActGroups]; accum
    static constexpr int nbars = 2 * C::kPkGroups + 2 * C::kWGroups + 2 * C::kActGroups + 1;
    static constexpr int misc = bars + 8 * nbars;
    static constexpr int total = misc + 16;
    static constexpr int kTmemCols = R * H * BN <= 128 ? 128 : R * H * BN <= 256 ? 256 : 512;
};

// Re-lays tiled (or row-major) bf16 activations [rows, K] into blocks of [128 rows x 32 K] = 8 KiB, each in the
// canonical K-major no-swizzle operand layout (8x8 core matrices of 128 contiguous bytes, K-groups 128 B apart,
// row-groups 512 B apart), ordered [row block of 128*R][K block][sub-block of 128 rows]. One thread moves 16 bytes.
__global__ void relayout_activations(const uint16_t *__restrict__ src, uint4 *__restrict__ dst, int64_t rows, int64_t K, int R,
                                     int a_row_major) {
    const int64_t nchunks = rows * K / 8;
    const int64_t nkb = K / BK, Kt = K / 32;
    for (int64_t d = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; d < nchunks; d += (int64_t)gridDim.x * blockDim.x) {
        const int64_t sub = d >> 9;            // 512 chunks per 8 KiB sub-block
        const int c = (int)(d & 511);
        const int mc = c >> 5, kc = (c >> 3) & 3, mr = c & 7;
        const int64_t rr = sub % R, kb = (sub / R) % nkb, mb = sub / (R * nkb);
        const int64_t m = (mb * R + rr) * BMS + mc * 8 + mr;
        const int64_t k = kb * BK + kc * 8;
        int64_t off;
        if (a_row_major)
            off = m * K + k;
        else
            off = ((m >> 5) * Kt + (k >> 5)) * 1024 + 256 * (2 * (int)((m & 31) >> 4) + (int)((k & 31) >> 4)) + 16 * (int)(m & 15) + (int)(k & 15);
        dst[d] = __ldg(reinterpret_cast<const uint4 *>(src + off));
    }
}

// Same expansion as the decode kernel: 16 codes sharing exponent E -> eight packed bf16 pairs (subnormal trick, one
// packed multiply by 2^min(E,127); BIG adds the factor 2^(E-127) for rows whose largest magnitude is 2 or more).
template <int FMT, bool BIG>
__device__ __forceinline__ void expand_row(const uint32_t *codes, uint32_t E, uint32_t (&out)[8]) {
    const uint32_t sb = (min(E, 127u) + 127u) << 7;
    const uint32_t scale2 = sb | (sb << 16);
    const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162 *>(&scale2);
    if (FMT == TTB_BFLOAT8_B) {
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t x = __byte_perm(codes[wi], 0u, h ? 0x3322u : 0x1100u) & 0x807f807fu;
                __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&x), s2);
                out[2 * wi + h] = *reinterpret_cast<uint32_t *>(&v);
            }
        }
    } else {
#pragma unroll
        for (int wi = 0; wi < 2; ++wi) {
            const uint32_t ev = (codes[wi] << 4) & 0xf0f0f0f0u, od = codes[wi] & 0xf0f0f0f0u;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t x = __byte_perm(ev, od, (uint32_t)(q | (q << 4) | ((4 + q) << 8) | ((4 + q) << 12))) & 0x80708070u;
                __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&x), s2);
                out[4 * wi + q] = *reinterpret_cast<uint32_t *>(&v);
            }
        }
    }
    if (BIG) {
        const uint32_t tb = max(min(E, 254u), 127u) << 7;
        const uint32_t t2v = tb | (tb << 16);
        const __nv_bfloat162 t2 = *reinterpret_cast<const __nv_bfloat162 *>(&t2v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&out[i]), t2);
            out[i] = *reinterpret_cast<uint32_t *>(&v);
        }
    }
}

struct PrefillArgs {
    const uint8_t *w;       // packed weight tiles [K, N]
    const uint8_t *x;       // re-laid activations (relayout_activations)
    const uint16_t *bias;
    void *out;
    int64_t K, N, rows;
    int Nt, nkb;
    int act, out_dtype, out_row_major;
    int *status;
    int x_R;            // 128-row sub-blocks per row block in the re-laid activations (the R relayout_activations was given)
    int64_t col_base;   // first weight / output column this launch covers (a multiple of 256)
};

template <int FMT, int R, int H>
__global__ void __launch_bounds__(kThreads, 1) matmul_prefill_kernel(const PrefillArgs p) {
    using L = Layout<FMT, R, H>;
    using C = Cfg<H>;
    constexpr int TB = Pk<FMT>::kTileBytes;
    constexpr int kGroup = C::kGroup, kPkGroups = C::kPkGroups, kWGroups = C::kWGroups, kActGroups = C::kActGroups;
    constexpr int kWStageBytes = C::kWStageBytes;
    constexpr int BNB = H * BN;   // block width in columns
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + L::bars;
    auto full_pk = [&](int s) { return bar0 + 8u * s; };
    auto empty_pk = [&](int s) { return bar0 + 8u * (kPkGroups + s); };
    auto full_w = [&](int s) { return bar0 + 8u * (2 * kPkGroups + s); };
    auto empty_w = [&](int s) { return bar0 + 8u * (2 * kPkGroups + kWGroups + s); };
    auto full_x = [&](int s) { return bar0 + 8u * (2 * kPkGroups + 2 * kWGroups + s); };
    auto empty_x = [&](int s) { return bar0 + 8u * (2 * kPkGroups + 2 * kWGroups + kActGroups + s); };
    const uint32_t accum_bar = bar0 + 8u * (2 * kPkGroups + 2 * kWGroups + 2 * kActGroups);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::misc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::misc + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // row blocks vary fastest across the grid: the blocks that share a weight column block run together, so the packed
    // tiles are read from HBM once and served to the other row blocks from L2
    const int mblock = blockIdx.x, ntile = blockIdx.y;
    const int nit = p.nkb;
    const int ngroups = (nit + kGroup - 1) / kGroup;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPkGroups; ++s) {
            mbar_init(full_pk(s), 1);
            mbar_init(empty_pk(s), C::kMembers);
        }
        for (int s = 0; s < kWGroups; ++s) {
            mbar_init(full_w(s), C::kMembers);
            mbar_init(empty_w(s), 1);
        }
        for (int s = 0; s < kActGroups; ++s) {
            mbar_init(full_x(s), 1);
            mbar_init(empty_x(s), 1);
        }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
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

    if (warp == kProducerWarp) {
        // ---------------- producer: packed weight tiles and activation blocks -> shared memory ----------------
        // (the whole warp walks the loop, so that addresses stay warp-uniform values; one elected lane issues)
        {
            const bool leader = elect_one();
            const uint8_t *wsrc = p.w + ((p.col_base >> 5) + (int64_t)ntile * 4 * H) * TB;
            const int64_t w_step = (int64_t)p.Nt * TB;
            // this block's activation sub-blocks inside the re-laid buffer (laid out for row blocks of p.x_R sub-blocks)
            const int64_t sub0 = (int64_t)mblock * R;
            const int64_t x_stage_step = (int64_t)p.x_R * kActSubBytes;
            const uint8_t *xsrc = p.x + ((sub0 / p.x_R) * p.nkb) * x_stage_step + (sub0 % p.x_R) * kActSubBytes;
            const bool x_contiguous = p.x_R == R;
            int gs = 0, gx = 0;
            uint32_t phs = 0, phx = 0;
            for (int g = 0; g < ngroups; ++g) {
                const int r = min(kGroup, nit - g * kGroup);  // stages in this group (the last one may be short)
                if (!__all_sync(0xffffffffu, mbar_wait(empty_x(gx), phx ^ 1, abort_flag, p.status, 21))) { ok = false; break; }
                if (leader) {
                    mbar_arrive_expect_tx(full_x(gx), r * L::kActStageBytes);
                    if (x_contiguous) {
                        // the r activation blocks of the group are adjacent in the re-laid buffer
                        bulk_g2s_plain(sbase + L::x + gx * kGroup * L::kActStageBytes, xsrc, r * L::kActStageBytes, full_x(gx));
                    } else {
                        for (int j = 0; j < r; ++j)
                            bulk_g2s_plain(sbase + L::x + (gx * kGroup + j) * L::kActStageBytes, xsrc + j * x_stage_step, L::kActStageBytes,
                                           full_x(gx));
                    }
                }
                xsrc += r * x_stage_step;
                if (!__all_sync(0xffffffffu, mbar_wait(empty_pk(gs), phs ^ 1, abort_flag, p.status, 22))) { ok = false; break; }
                if (leader) {
                    mbar_arrive_expect_tx(full_pk(gs), r * L::kPkStageBytes);
                    for (int j = 0; j < r; ++j)
                        bulk_g2s_plain(sbase + L::pk + (gs * kGroup + j) * L::kPkStageBytes, wsrc + j * w_step, L::kPkStageBytes, full_pk(gs));
                }
                wsrc += r * w_step;
                if (++gs == kPkGroups) { gs = 0; phs ^= 1; }
                if (++gx == kActGroups) { gx = 0; phx ^= 1; }
            }
        }
    } else if (warp == kMmaWarp) {
        // ---------------- MMA issuer (warp-uniform, one elected lane issues) ----------------
        {
            const bool leader = elect_one();
            constexpr uint32_t idesc = instr_desc_bf16_f32(BMS, BNB, /*a_mn_major=*/false, /*b_mn_major=*/true);
            const uint64_t x_desc0 = smem_desc_noswizzle(sbase + L::x, kX_LBO, kX_SBO);
            const uint64_t w_desc0 = smem_desc_noswizzle(sbase + L::w, kW_LBO, kW_SBO);
            const uint32_t x_lo0 = (uint32_t)x_desc0, x_hi = (uint32_t)(x_desc0 >> 32);
            const uint32_t w_lo0 = (uint32_t)w_desc0, w_hi = (uint32_t)(w_desc0 >> 32);
            auto mk = [](uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; };
            int gw = 0, gx = 0;
            uint32_t phw = 0, phx = 0;
            for (int g = 0; g < ngroups; ++g) {
                const int r = min(kGroup, nit - g * kGroup);
                if (leader)
                    for (int j = r * H; j < C::kMembers; ++j) mbar_arrive(full_w(gw));  // stand in for the stages a short last group lacks
                if (!__all_sync(0xffffffffu, mbar_wait(full_x(gx), phx, abort_flag, p.status, 23) && mbar_wait(full_w(gw), phw, abort_flag, p.status, 24))) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t x_lo = x_lo0 + (uint32_t)gx * ((kGroup * L::kActStageBytes) >> 4);
                const uint32_t w_lo = w_lo0 + (uint32_t)gw * ((kGroup * kWStageBytes) >> 4);
#pragma unroll
                for (int j = 0; j < kGroup; ++j) {
                    if (j < r) {
#pragma unroll
                        for (int k16 = 0; k16 < BK / 16; ++k16) {
#pragma unroll
                            for (int rr = 0; rr < R; ++rr)
                                if (leader) mma_bf16_ss(tmem_base + (uint32_t)(rr * BNB),
                                            mk(x_lo + ((j * L::kActStageBytes + rr * kActSubBytes + k16 * 2 * kX_LBO) >> 4), x_hi),
                                            mk(w_lo + ((j * kWStageBytes + k16 * 2 * kW_LBO) >> 4), w_hi), idesc,
                                            j > 0 || k16 > 0 || g > 0);
                        }
                    }
                }
                if (leader) {
                    mma_commit(empty_w(gw));
                    mma_commit(empty_x(gx));
                }
                if (++gw == kWGroups) { gw = 0; phw ^= 1; }
                if (++gx == kActGroups) { gx = 0; phx ^= 1; }
            }
            if (ok && leader) mma_commit(accum_bar);
        }
    } else if ((warp & 3) != 0) {
        // ---------------- expand warps: packed codes -> bf16 weights in shared memory (B operand) ----------------
        const int ew = (warp >> 2) * 3 + (warp & 3) - 1;
        const int lane_pk = lane * (FMT == TTB_BFLOAT8_B ? 16 : 8);
        const int lane_w = ((lane & 15) >> 3) * kW_LBO + (lane >> 4) * 2 * kW_SBO + (lane & 7) * 16;
        // team ew / kMembers takes every kTeams-th group; within a group this warp expands half `hh` of stage `st`
        const int member = ew % C::kMembers, st = member / H, hh = member % H;
        for (int g = ew / C::kMembers; ew < C::kTeams * C::kMembers && g < ngroups; g += C::kTeams) {
            const int it = g * kGroup + st;
            if (it >= nit) break;  // short last group: the MMA issuer arrives in this warp's place
            const int gs = g % kPkGroups, gw = g % kWGroups;
            const int s = gs * kGroup + st, t = gw * kGroup + st;
            const uint32_t phs = (g / kPkGroups) & 1, phw = (g / kWGroups) & 1;
            int good = 1;
            if (lane == 0)
                good = mbar_wait(empty_w(gw), phw ^ 1, abort_flag, p.status, 25) && mbar_wait(full_pk(gs), phs, abort_flag, p.status, 26);
            good = __shfl_sync(0xffffffffu, good, 0);
            if (!good) { ok = false; break; }
            const uint8_t *pst = smem + L::pk + s * L::kPkStageBytes + hh * Pk<FMT>::kRunBytes;
            uint8_t *const wst = smem + L::w + t * kWStageBytes + hh * (BN * BK * 2) + lane_w;
            uint32_t Es[8];
            uint32_t codes[8][4];
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) {
                // face row rr * 32 + lane of the stage: tile rr / 2, faces 2 * (rr & 1) (+1 for lanes 16-31), row lane & 15
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
                    // k_local = (rr & 1) * 16 + (lane & 15), n_local = (rr / 2) * 32 + (lane / 16) * 16
                    uint8_t *dst = wst + (rr & 1) * 2 * kW_LBO + (rr >> 1) * 4 * kW_SBO;
                    *reinterpret_cast<uint4 *>(dst) = make_uint4(vals[0], vals[1], vals[2], vals[3]);
                    *reinterpret_cast<uint4 *>(dst + kW_SBO) = make_uint4(vals[4], vals[5], vals[6], vals[7]);
                }
            };
            if (__any_sync(0xffffffffu, emax > 127u))
                expand_stage(std::true_type{});
            else
                expand_stage(std::false_type{});
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(full_w(gw));
                mbar_arrive(empty_pk(gs));
            }
        }
    }

    if (warp < 8) {
        // ---------------- epilogue: warps 0..7; TMEM lanes (rows) 32 * (warp % 4) .., column half warp / 4 ----------------
        {
            int good = ok ? 1 : 0;
            good = __shfl_sync(0xffffffffu, good, 0);   // lane 0 ran the single-thread roles
            if (lane == 0 && good) good = mbar_wait(accum_bar, 0, abort_flag, p.status, 27);
            ok = __shfl_sync(0xffffffffu, good, 0) != 0;
        }
        tc_fence_after_sync();
        const int quad = warp & 3, half = warp >> 2;
        if (ok) {
#pragma unroll 1
            for (int rr = 0; rr < R; ++rr) {
                const int64_t row = ((int64_t)mblock * R + rr) * BMS + quad * 32 + lane;
#pragma unroll 1
                for (int cc = 0; cc < BNB / 32; ++cc) {
                    const int col0 = half * (BNB / 2) + cc * 16;
                    const int64_t n0 = p.col_base + (int64_t)ntile * BNB + col0;
                    uint32_t r[16];
                    tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(rr * BNB + col0), r);
                    tmem_ld_wait();
                    float v[16];
                    TTB_DISPATCH_ACT(p.act, {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            float y = __uint_as_float(r[j]);
                            if (p.bias) y += bias_at(p.bias, n0 + j);
                            v[j] = apply_activation_t<ACT>(y);
                        }
                    });
                    // 16 consecutive columns of one row: one face row when tiled, contiguous either way
                    const int64_t off = p.out_row_major ? row * p.N + n0 : tiled_offset(row, n0, p.Nt);
                    if (p.out_dtype == TTB_FLOAT32) {
                        float4 *o = reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.out) + off);
#pragma unroll
                        for (int j = 0; j < 4; ++j) o[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    } else {
                        uint32_t h[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            h[j] = (uint32_t)f32_to_bf16_bits(v[2 * j]) | ((uint32_t)f32_to_bf16_bits(v[2 * j + 1]) << 16);
                        uint4 *o = reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(p.out) + off);
                        o[0] = make_uint4(h[0], h[1], h[2], h[3]);
                        o[1] = make_uint4(h[4], h[5], h[6], h[7]);
                    }
                }
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

template <int FMT, int R, int H>
int32_t launch_one(const PrefillArgs &p, dim3 grid, cudaStream_t stream) {
    constexpr int smem_bytes = Layout<FMT, R, H>::total + 128;
    static_assert(smem_bytes <= 232448, "shared memory budget");
    static bool configured[64] = {};
    int dev = 0;
    TTB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        TTB_CUDA_TRY(cudaFuncSetAttribute(matmul_prefill_kernel<FMT, R, H>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        configured[dev] = true;
    }
    matmul_prefill_kernel<FMT, R, H><<<grid, kThreads, smem_bytes, stream>>>(p);
    TTB_LAUNCH_CHECK("matmul_prefill");
    return TTB_OK;
}
}  // namespace

bool prefill_supported(int w_dtype, int64_t rows, int64_t K, int64_t N) {
    return (w_dtype == TTB_BFLOAT8_B || w_dtype == TTB_BFLOAT4_B) && rows >= 512 && rows % BMS == 0 && K % BK == 0 && N % BN == 0 &&
           N / BN <= 65535;
}

// Scratch for the re-laid activations.
// The head of a matmul workspace (64 KiB of arrival counters + 16 MiB of accumulation tiles) belongs to the split-K
// decode kernels and must stay zero; the re-laid activations go behind it.
static constexpr int64_t kReservedHead = 65536 + (16 << 20);
int64_t prefill_workspace_bytes(int64_t rows, int64_t K) { return kReservedHead + rows * K * 2; }

int32_t launch_matmul_prefill(const void *a, const void *w, int w_dtype, const void *bias, void *out, int out_dtype, int64_t rows,
                              int64_t K, int64_t N, int act, int flags, void *workspace, int64_t workspace_bytes, int *status,
                              cudaStream_t stream) {
    const int64_t need = prefill_workspace_bytes(rows, K);
    if (!workspace || workspace_bytes < need)
        return fail(TTB_E_WORKSPACE, "ttb_matmul: this shape needs %lld bytes of workspace, got %lld", (long long)need,
                    (long long)workspace_bytes);
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return fail(TTB_E_INVALID, "ttb_matmul: workspace must be 256-byte aligned");
    const int R = rows % (2 * BMS) == 0 ? 2 : 1;
    {
        const int64_t nchunks = rows * K / 8;
        const int blocks = (int)((nchunks + 255) / 256 < 148 * 16 ? (nchunks + 255) / 256 : 148 * 16);
        relayout_activations<<<blocks, 256, 0, stream>>>((const uint16_t *)a, (uint4 *)((uint8_t *)workspace + kReservedHead), rows, K, R,
                                                         (flags & TTB_MM_A_ROW_MAJOR) != 0);
        TTB_LAUNCH_CHECK("relayout_activations");
    }
    PrefillArgs p;
    p.w = (const uint8_t *)w; p.x = (const uint8_t *)workspace + kReservedHead; p.bias = (const uint16_t *)bias; p.out = out;
    p.K = K; p.N = N; p.rows = rows; p.Nt = (int)(N / 32); p.nkb = (int)(K / BK);
    p.act = act; p.out_dtype = out_dtype; p.out_row_major = (flags & TTB_MM_OUT_ROW_MAJOR) != 0;
    p.status = status;
    p.x_R = R; p.col_base = 0;
    // 256-column blocks halve how often the activations are fetched from L2 (once per block column): that traffic, not the
    // tensor pipe, bounds the 128-column form (7.5 GB per launch for the Llama MLP shape).
    const int H = (R == 2 && N % (2 * BN) == 0) ? 2 : 1;
    dim3 grid((unsigned)(rows / (BMS * R)), (unsigned)(N / (BN * H)));
    // Whole waves: one block per SM runs at a time, so a handful of blocks left over after the last full wave would cost a
    // whole block time (8 of 896 blocks on the Llama MLP shape: 14 %). The column blocks that do not fill a wave are
    // given to a second launch with quarter-size blocks (128 x 128), whose tail is a quarter as long.
    int dev = 0, kSms = 148;   // multiprocessors of the device at hand
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&kSms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || kSms <= 0) kSms = 148;
    const int64_t nblocks = (int64_t)grid.x * grid.y;
    if (H == 2 && nblocks > kSms && nblocks % kSms != 0 && (nblocks % kSms) * 4 < kSms) {
        const unsigned cols_main = (unsigned)((nblocks / kSms) * kSms / grid.x);   // column blocks of the main launch
        if (cols_main > 0 && cols_main < grid.y) {
            dim3 gmain(grid.x, cols_main);
            int32_t rc = w_dtype == TTB_BFLOAT8_B ? launch_one<TTB_BFLOAT8_B, 2, 2>(p, gmain, stream) : launch_one<TTB_BFLOAT4_B, 2, 2>(p, gmain, stream);
            if (rc != TTB_OK) return rc;
            PrefillArgs q = p;
            q.col_base = (int64_t)cols_main * 2 * BN;
            dim3 gtail((unsigned)(rows / BMS), (unsigned)((N - q.col_base) / BN));
            return w_dtype == TTB_BFLOAT8_B ? launch_one<TTB_BFLOAT8_B, 1, 1>(q, gtail, stream) : launch_one<TTB_BFLOAT4_B, 1, 1>(q, gtail, stream);
        }
    }
    if (w_dtype == TTB_BFLOAT8_B) {
        if (H == 2) return launch_one<TTB_BFLOAT8_B, 2, 2>(p, grid, stream);
        return R == 2 ? launch_one<TTB_BFLOAT8_B, 2, 1>(p, grid, stream) : launch_one<TTB_BFLOAT8_B, 1, 1>(p, grid, stream);
    }
    if (H == 2) return launch_one<TTB_BFLOAT4_B, 2, 2>(p, grid, stream);
    return R == 2 ? launch_one<TTB_BFLOAT4_B, 2, 1>(p, grid, stream) : launch_one<TTB_BFLOAT4_B, 1, 1>(p, grid, stream);
}

}  // namespace ttb
