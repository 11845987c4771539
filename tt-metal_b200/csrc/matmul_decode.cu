// Weight-streaming matmul for small row counts (decode): out[rows, N] = act(a[rows, K] x W[K, N] + bias)
// with W in packed bfloat8_b / bfloat4_b tiles, rows in {32, 64, 128} per block.
//
// The kernel is bound by reading W once from HBM (1.0625 or 0.5625 bytes per weight), so everything is
// organised around keeping many weight bytes in flight per SM and spending few instructions per weight:
//   * "swap-AB": the tensor-core M dimension (128) runs over weight columns, the MMA N dimension over the
//     activation rows, so a 32-row batch fills the MMA instead of wasting three quarters of it;
//   * a producer thread streams packed tiles (a run of four tiles = 4352 / 2304 contiguous bytes per stage)
//     into a 16-deep shared-memory ring with cp.async.bulk, each stage completing on an mbarrier;
//   * eight expand warps each own every eighth stage: one lane polls the barriers, the warp expands the 4096
//     packed codes of the stage to bf16 (exact: sign + 7-bit mantissa under an 8-bit exponent fits bf16) straight
//     into the tensor cores' canonical no-swizzle operand layout and stages the activation K-block next to it.
//     Eight stages are therefore expanded concurrently, which hides barrier and shared-memory latency;
//   * one thread issues tcgen05.mma (kind::f16, bf16 x bf16 -> fp32 in TMEM); tcgen05.commit hands operand
//     stages back to their expand warp;
//   * the expand warps then read the accumulator with tcgen05.ld and finish: either bias + activation +
//     store, or - when K is split over several blocks so that every SM streams - an fp32 partial into scratch,
//     where the last block to arrive for an output tile adds the partials in a fixed order and finishes.
// Every mbarrier wait is bounded; a wait that runs out raises a status word instead of hanging.
#include <type_traits>

#include "decode_common.cuh"

namespace ttb {

__device__ int g_status_word = 0;

namespace {

using namespace ptx;

constexpr int BN = 128;           // weight columns per block (UMMA M)
constexpr int BK = 32;            // K per pipeline stage (one row of four tiles)
// Twelve warps. A warp's scheduler is warp % 4: the single-thread roles (warp 0 producer, warps 4 and 8 MMA issuers)
// share scheduler 0, so the MMA issuers never compete with expand warps for issue slots.
// The nine warps with warp % 4 != 0 expand; warps 0..7 run the epilogue (TMEM lane quadrant = warp % 4).
constexpr int kWarps = 12;
constexpr int kThreadsDecode = 32 * kWarps;
constexpr int kExpandWarps = 9;
constexpr int kProducerWarp = 0, kMmaWarp = 4, kMmaWarp2 = 8;
constexpr int kEpilogueThreads = 256;
// Stages are handled in groups of three consecutive K-blocks, one per warp of an expand-warp triplet, with one
// mbarrier per group: the producer and the MMA issuer then pay their per-iteration latencies (barrier wait,
// tcgen05 fence, commit) once per three stages.
constexpr int kGroup = 3;
constexpr int kPkGroups = 5;                    // packed ring: 15 stages
constexpr int kPkStages = kGroup * kPkGroups;
template <int NB>
struct Ab {
    // bf16 operand ring (per stage: A 8 KiB + B NB*64 bytes), in groups of three stages
    static constexpr int kGroups = NB == 128 ? 3 : 4;
    static constexpr int kStages = kGroup * kGroups;
};
constexpr int kAStageBytes = BN * BK * 2;       // 8 KiB
constexpr uint32_t kA_LBO = 128, kA_SBO = 512;   // A (weights, N-contiguous): the four K-groups of a stage adjacent, N-groups 512 B apart
constexpr uint32_t kB_LBO = 128, kB_SBO = 512;   // B (activations, K-contiguous): K-groups adjacent, row-groups 512 B apart

template <int FMT>
struct Pk {
    static constexpr int kTileBytes = FMT == TTB_BFLOAT8_B ? kBfp8TileBytes : kBfp4TileBytes;
    static constexpr int kStageBytes = 4 * kTileBytes;
};

template <int FMT, int NB>
struct SmemLayout {
    static constexpr int kBStageBytes = NB * BK * 2;
    static constexpr int pk = 0;
    static constexpr int a = pk + kPkStages * Pk<FMT>::kStageBytes;
    static constexpr int kAbStages = Ab<NB>::kStages;
    static constexpr int b = a + kAbStages * kAStageBytes;
    static constexpr int bars = b + kAbStages * kBStageBytes;
    // barriers: full_pk[kPkGroups], empty_pk[kPkGroups], full_ab[kAbGroups], empty_ab[kAbGroups], accum
    static constexpr int kAbGroups = Ab<NB>::kGroups;
    static constexpr int nbars = 2 * kPkGroups + 2 * kAbGroups + 1;
    static constexpr int misc = bars + 8 * nbars;  // tmem base (4), abort flag (4), last-block flag (4)
    static constexpr int total = misc + 16;
};

// Expands one face row (16 codes sharing exponent E) into 16 bf16 values, returned as eight packed pairs.
// value = +-m * 2^(E - 133) (bfloat8_b) or +-m * 2^(E - 129) (bfloat4_b). A bf16 with a zero exponent field and
// mantissa bits m is the subnormal m * 2^-133, so the halfword (sign << 15) | m (bfloat8_b) or
// (sign << 15) | (m << 4) (bfloat4_b) already is the weight up to the factor 2^E: one packed multiply by the
// power of two finishes it, exactly. 2^E is a bf16 only up to E = 127 (rows whose largest magnitude is below 2);
// larger exponents take a second multiply (BIG; chosen per stage by a warp vote so that the common path has no
// divergent branch).
template <int FMT, bool BIG>
__device__ __forceinline__ void expand_row(const uint32_t *codes, uint32_t E, uint32_t (&out)[8]) {
    const uint32_t e1 = min(E, 127u);
    const uint32_t sb = (e1 + 127u) << 7;
    const uint32_t scale2 = sb | (sb << 16);
    const __nv_bfloat162 s2 = *reinterpret_cast<const __nv_bfloat162 *>(&scale2);
    if (FMT == TTB_BFLOAT8_B) {
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
            const uint32_t w = codes[wi];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t x = __byte_perm(w, 0u, h ? 0x3322u : 0x1100u) & 0x807f807fu;  // [c, c] per halfword -> sign | mantissa
                __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&x), s2);
                out[2 * wi + h] = *reinterpret_cast<uint32_t *>(&v);
            }
        }
    } else {
#pragma unroll
        for (int wi = 0; wi < 2; ++wi) {
            const uint32_t w = codes[wi];
            const uint32_t ev = (w << 4) & 0xf0f0f0f0u, od = w & 0xf0f0f0f0u;  // even / odd elements: [s m m m 0 0 0 0] per byte
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                uint32_t x = __byte_perm(ev, od, (uint32_t)(p | (p << 4) | ((4 + p) << 8) | ((4 + p) << 12))) & 0x80708070u;
                __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&x), s2);
                out[4 * wi + p] = *reinterpret_cast<uint32_t *>(&v);
            }
        }
    }
    if (BIG) {
        const uint32_t tb = max(min(E, 254u), 127u) << 7;  // 2^(E - 127), 1 for rows at or below 127
        const uint32_t t2v = tb | (tb << 16);
        const __nv_bfloat162 t2 = *reinterpret_cast<const __nv_bfloat162 *>(&t2v);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            __nv_bfloat162 v = __hmul2(*reinterpret_cast<__nv_bfloat162 *>(&out[i]), t2);
            out[i] = *reinterpret_cast<uint32_t *>(&v);
        }
    }
}

template <int FMT, int NB>
__global__ void __launch_bounds__(kThreadsDecode, 1) matmul_decode_kernel(const DecodeArgs p) {
    using L = SmemLayout<FMT, NB>;
    constexpr int TB = Pk<FMT>::kTileBytes;
    constexpr int kAcc = BK / 16;  // one accumulator per K step of a stage (two); summed in the epilogue
    constexpr int kTmemCols = NB * kAcc < 32 ? 32 : NB * kAcc;
    constexpr int kAbGroups = Ab<NB>::kGroups;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar0 = sbase + L::bars;
    auto full_pk = [&](int s) { return bar0 + 8u * s; };
    auto empty_pk = [&](int s) { return bar0 + 8u * (kPkGroups + s); };
    auto full_ab = [&](int s) { return bar0 + 8u * (2 * kPkGroups + s); };
    auto empty_ab = [&](int s) { return bar0 + 8u * (2 * kPkGroups + kAbGroups + s); };
    const uint32_t accum_bar = bar0 + 8u * (2 * kPkGroups + 2 * kAbGroups);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L::misc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::misc + 4);
    volatile int *last_flag = reinterpret_cast<volatile int *>(smem + L::misc + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntile = blockIdx.x, split = blockIdx.y, rchunk = blockIdx.z;
    const int kb0 = split * p.kb_per_split;
    const int kb1 = min(p.nkb, kb0 + p.kb_per_split);
    const int nit = kb1 - kb0;
    const int ngroups = (nit + kGroup - 1) / kGroup;
    const int64_t row0 = (int64_t)rchunk * NB;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPkGroups; ++s) {
            mbar_init(full_pk(s), 1);
            mbar_init(empty_pk(s), kGroup);
        }
        for (int s = 0; s < kAbGroups; ++s) {
            mbar_init(full_ab(s), kGroup);
            mbar_init(empty_ab(s), 2);   // one commit from each of the two MMA issuers
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
    // The next kernel on the stream may start its own set-up and weight streaming while this grid drains. Only the packed
    // weights are read before grid_dep_wait(): activations, bias, scratch and the output wait for the previous grid.
    grid_dep_launch();

    if (warp == kProducerWarp) {
        // ---------------- producer: packed weight tiles -> shared-memory ring ----------------
        if (lane == 0) {
            const uint64_t policy = l2_policy_evict_first();
            const uint8_t *src = p.w + ((int64_t)kb0 * p.Nt + (int64_t)ntile * 4) * TB;
            const int64_t src_step = (int64_t)p.Nt * TB;
            int gs = 0;
            uint32_t ph = 0;
            for (int g = 0; g < ngroups; ++g) {
                const int r = min(kGroup, nit - g * kGroup);  // stages in this group (the last one may be short)
                if (!mbar_wait(empty_pk(gs), ph ^ 1, abort_flag, p.status, 1)) { ok = false; break; }
                mbar_arrive_expect_tx(full_pk(gs), r * Pk<FMT>::kStageBytes);
                for (int j = 0; j < r; ++j) {
                    bulk_g2s(sbase + L::pk + (gs * kGroup + j) * Pk<FMT>::kStageBytes, src, 4 * TB, full_pk(gs), policy);
                    src += src_step;
                }
                if (++gs == kPkGroups) { gs = 0; ph ^= 1; }
            }
        }
    } else if (warp == kMmaWarp || warp == kMmaWarp2) {
        // ---------------- MMA issuers: warp 4 issues the first K step of every stage (accumulator 0), warp 8 the second
        // (accumulator 1). The two instruction streams are independent, which doubles the rate at which MMAs are issued.
        const int k16 = warp == kMmaWarp ? 0 : 1;
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc_bf16_f32(BN, NB, /*a_mn_major=*/true, /*b_mn_major=*/false);
            // descriptors differ between stages and K steps only in the 14-bit start-address field (units of 16 B)
            const uint64_t a_desc0 = smem_desc_noswizzle(sbase + L::a, kA_LBO, kA_SBO);
            const uint64_t b_desc0 = smem_desc_noswizzle(sbase + L::b, kB_LBO, kB_SBO);
            // The loop below is one thread's dependent instruction stream, so it is kept short: descriptors are
            // formed by a 32-bit add into the low word, the accumulator of each K step is fixed at compile time.
            const uint32_t a_lo0 = (uint32_t)a_desc0, a_hi = (uint32_t)(a_desc0 >> 32);
            const uint32_t b_lo0 = (uint32_t)b_desc0, b_hi = (uint32_t)(b_desc0 >> 32);
            auto mk = [](uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; };
            const uint32_t d_tmem = tmem_base + (uint32_t)(k16 * NB);
            int gt = 0;
            uint32_t ph = 0;
            for (int g = 0; g < ngroups; ++g) {
                const int r = min(kGroup, nit - g * kGroup);
                if (k16 == 0)
                    for (int j = r; j < kGroup; ++j) mbar_arrive(full_ab(gt));  // stand in for the stages a short last group lacks
                if (!mbar_wait(full_ab(gt), ph, abort_flag, p.status, 2)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t a_lo = a_lo0 + (uint32_t)gt * ((kGroup * kAStageBytes) >> 4) + (uint32_t)k16 * ((2 * kA_LBO) >> 4);
                const uint32_t b_lo = b_lo0 + (uint32_t)gt * ((kGroup * L::kBStageBytes) >> 4) + (uint32_t)k16 * ((2 * kB_LBO) >> 4);
#pragma unroll
                for (int j = 0; j < kGroup; ++j) {
                    if (j < r)
                        mma_bf16_ss(d_tmem, mk(a_lo + ((j * kAStageBytes) >> 4), a_hi), mk(b_lo + ((j * L::kBStageBytes) >> 4), b_hi), idesc,
                                    j > 0 || g > 0);
                }
                mma_commit(empty_ab(gt));
                if (++gt == kAbGroups) { gt = 0; ph ^= 1; }
            }
            if (ok) mma_commit(accum_bar);
        }
    } else if ((warp & 3) != 0) {
        // ---------------- expand warps: packed -> bf16 operands ----------------
        const int ew = (warp >> 2) * 3 + (warp & 3) - 1;
        constexpr int kActChunks = NB / 8;  // 16-byte activation chunks per lane per K-block (NB rows x 4 chunks)
        uint4 act_regs[kActChunks];
        const uint16_t *act_src[kActChunks];
#pragma unroll
        for (int j = 0; j < kActChunks; ++j) {
            const int c = j * 32 + lane;
            act_src[j] = p.a + act_chunk_base(p, row0 + c % NB, c / NB) + (int64_t)kb0 * act_chunk_step(p);
        }
        const int act_step = act_chunk_step(p);
        grid_dep_wait();
        if (p.wait_arrived) {
            // activations gathered from other GPUs: hold until every rank's slice has landed in this rank's copy
            int good = 1;
            if (lane == 0) good = peer_wait(p, abort_flag, 6) ? 1 : 0;
            if (!__shfl_sync(0xffffffffu, good, 0)) ok = false;
        }
        auto load_act = [&](int it) {
#pragma unroll
            for (int j = 0; j < kActChunks; ++j) act_regs[j] = __ldcg(reinterpret_cast<const uint4 *>(act_src[j] + (int64_t)it * act_step));
        };
        if (ok && ew < nit) load_act(ew);  // this warp's first stage is K-block ew (group ew / 3, member ew % 3)
        // lane-constant parts of the addressing: lanes 0-15 take the left face of a tile, 16-31 the right one
        const int lane_pk = lane * (FMT == TTB_BFLOAT8_B ? 16 : 8);
        const int lane_a = ((lane & 15) >> 3) * kA_LBO + (lane >> 4) * 2 * kA_SBO + (lane & 7) * 16;
        // triplet ew / 3 takes every third group; within a group this warp expands stage ew % 3
        for (int g = ew / kGroup; ok && g < ngroups; g += kExpandWarps / kGroup) {
            const int it = g * kGroup + ew % kGroup;
            if (it >= nit) break;  // short last group: the MMA issuer arrives in this warp's place
            const int gs = g % kPkGroups, gt = g % kAbGroups;
            const int s = gs * kGroup + ew % kGroup, t = gt * kGroup + ew % kGroup;
            const uint32_t phs = (g / kPkGroups) & 1, pht = (g / kAbGroups) & 1;
            int good = 1;
            if (lane == 0)
                good = mbar_wait(empty_ab(gt), pht ^ 1, abort_flag, p.status, 3) &&
                       mbar_wait(full_pk(gs), phs, abort_flag, p.status, 4);
            good = __shfl_sync(0xffffffffu, good, 0);
            if (!good) { ok = false; break; }
            const uint8_t *pst = smem + L::pk + s * Pk<FMT>::kStageBytes;
            uint8_t *const ast = smem + L::a + t * kAStageBytes + lane_a;
            uint8_t *const bst = smem + L::b + t * L::kBStageBytes;
            // all shared-memory loads of the stage first, so that their latency is paid once
            uint32_t Es[8];
            uint32_t codes[8][4];
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) {
                // face row R = rr * 32 + lane of the stage: tile rr / 2, faces 2 * (rr & 1) (+1 for lanes 16-31), row lane & 15
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
                    uint8_t *dst = ast + (rr & 1) * 2 * kA_LBO + (rr >> 1) * 4 * kA_SBO;
                    *reinterpret_cast<uint4 *>(dst) = make_uint4(vals[0], vals[1], vals[2], vals[3]);
                    *reinterpret_cast<uint4 *>(dst + kA_SBO) = make_uint4(vals[4], vals[5], vals[6], vals[7]);
                }
            };
            if (__any_sync(0xffffffffu, emax > 127u))
                expand_stage(std::true_type{});
            else
                expand_stage(std::false_type{});
            // activations of this K-block: loaded from global one turn ahead, stored last so the load has landed
#pragma unroll
            for (int j = 0; j < kActChunks; ++j) {
                const int c = j * 32 + lane;
                const int m = c % NB, kc = c / NB;
                *reinterpret_cast<uint4 *>(bst + (m >> 3) * kB_SBO + kc * kB_LBO + (m & 7) * 16) = act_regs[j];
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(full_ab(gt));
                mbar_arrive(empty_pk(gs));
            }
            if (it + kExpandWarps < nit) load_act(it + kExpandWarps);
        }
    }

    if (warp < 8) {
        // ---------------- epilogue: warps 0..7, TMEM lane quadrant warp % 4, column half warp / 4 ----------------
        const int tid = threadIdx.x;
        grid_dep_wait();
        uint16_t *const stage = p.ranks > 1 ? reinterpret_cast<uint16_t *>(smem + L::pk) : nullptr;   // the packed ring is idle by now
        if (p.ranks > 1 && tid == 0 && blockIdx.x + blockIdx.y + blockIdx.z == 0) *p.expected = *p.expected + p.launch_arrivals;
        {
            int good = ok ? 1 : 0;
            good = __shfl_sync(0xffffffffu, good, 0);   // lane 0 ran the single-thread roles
            if (lane == 0 && good && nit > 0) good = mbar_wait(accum_bar, 0, abort_flag, p.status, 5);
            ok = __shfl_sync(0xffffffffu, good, 0) != 0;
        }
        tc_fence_after_sync();
        const int quad = warp & 3;
        const int half = warp >> 2;
        constexpr int kColsPerWarp = NB / 2;
        const int64_t n = (int64_t)ntile * BN + quad * 32 + lane;
        const int tile_id = rchunk * gridDim.x + ntile;
        if (ok && nit > 0) {
#pragma unroll
            for (int cc = 0; cc < kColsPerWarp / 16; ++cc) {
                const int col0 = half * kColsPerWarp + cc * 16;
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0.0f;
#pragma unroll
                for (int ac = 0; ac < kAcc; ++ac) {
                    uint32_t r[16];
                    tmem_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(ac * NB + col0), r);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] += __uint_as_float(r[j]);
                }
                if (p.splits == 1) {
                    finish_and_store<NB>(p, v, row0, col0, n, stage);
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
#pragma unroll
                for (int cc = 0; cc < kColsPerWarp / 16; ++cc) {
                    const int col0 = half * kColsPerWarp + cc * 16;
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
                    finish_and_store<NB>(p, v, row0, col0, n, stage);
                }
                if (tid == 0) p.counters[tile_id] = 0;  // leave the scratch ready for the next launch
                if (p.ranks > 1) gather_send<NB>(p, stage, row0, ntile, tid, kEpilogueThreads);
            }
        } else if (p.ranks > 1) {
            // one decision for the whole block, so that every epilogue thread takes part in gather_send's barriers
            if (tid == 0) *last_flag = (*abort_flag == 0 && nit > 0) ? 1 : 0;
            asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
            if (*last_flag) gather_send<NB>(p, stage, row0, ntile, tid, kEpilogueThreads);
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
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

template <int FMT, int NB>
int32_t launch_one(const DecodeArgs &p, dim3 grid, bool overlap, cudaStream_t stream) {
    constexpr int smem_bytes = SmemLayout<FMT, NB>::total + 128;
    static bool configured[64] = {};
    int dev = 0;
    TTB_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
        TTB_CUDA_TRY(cudaFuncSetAttribute(matmul_decode_kernel<FMT, NB>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        configured[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kThreadsDecode);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    TTB_CUDA_TRY(cudaLaunchKernelEx(&cfg, matmul_decode_kernel<FMT, NB>, p));
    TTB_LAUNCH_CHECK("matmul_decode");
    return TTB_OK;
}

}  // namespace

// The head of the workspace holds one arrival counter per output tile; the partial sums follow.
static constexpr int64_t kCounterBytes = 65536;
// Workspace layout: [arrival counters, 64 KiB][accumulate-mode tiles, 16 MiB, zero between launches][ordered-mode
// partials / other scratch]. The compact layout (built-in scratch of the allocation-free entry point) has no middle part.
static constexpr int64_t kAccumBytes = 16 << 20;

int32_t launch_decode_tmem(const DecodeArgs &p, int nb, dim3 grid, bool overlap, cudaStream_t stream);

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

// Rows handled per block: the largest of 128 / 64 / 32 that divides `rows`.
static int decode_rows_per_block(int64_t rows) { return rows % 128 == 0 ? 128 : rows % 64 == 0 ? 64 : 32; }

bool decode_supported(int w_dtype, int64_t rows, int64_t K, int64_t N) {
    return (w_dtype == TTB_BFLOAT8_B || w_dtype == TTB_BFLOAT4_B) && rows > 0 && rows <= 256 && rows % 32 == 0 &&
           K % BK == 0 && N % BN == 0 && (N / BN) * (rows / 32) * 4 <= kCounterBytes;
}

// Chooses how many blocks share one output tile along K so that the grid fills the 148 SMs in whole waves.
void decode_plan(int64_t rows, int64_t K, int64_t N, int *splits_out, int *kb_per_split_out, int *tiles_out, int *nb_out) {
    const int nb = decode_rows_per_block(rows);
    const int tiles = (int)(N / BN) * (int)(rows / nb);
    const int nkb = (int)(K / BK);
    const int sms = 148;
    int best_s = 1;
    double best_cost = 1e30;
    for (int s = 1; s <= 32 && s <= nkb; ++s) {
        const int kbps = (nkb + s - 1) / s;
        const int real_s = (nkb + kbps - 1) / kbps;
        if (real_s != s) continue;
        if (s > 1 && kbps < 16) break;
        const int blocks = tiles * s;
        const int waves = (blocks + sms - 1) / sms;
        // time model in units of one K-block: each wave costs its blocks' K-blocks plus a fixed fill/drain
        // overhead; split partials add a small reduction cost.
        // in units of one K-block's streaming time (~0.16 us): a wave costs ~4 us to fill and drain, the last block of a
        // tile spends ~0.25 us per partial on the reduction
        const double cost = waves * (kbps + 25.0) + (s > 1 ? 6.0 + 1.5 * s : 0.0);
        if (cost < best_cost) { best_cost = cost; best_s = s; }
    }
    const int kbps = (nkb + best_s - 1) / best_s;
    *splits_out = (nkb + kbps - 1) / kbps;
    *kb_per_split_out = kbps;
    *tiles_out = tiles;
    *nb_out = nb;
}

// Bytes of the ordered-mode partials (0 when K is not split).
static int64_t decode_partial_bytes(int64_t rows, int64_t K, int64_t N) {
    int s, kbps, tiles, nb;
    decode_plan(rows, K, N, &s, &kbps, &tiles, &nb);
    return s == 1 ? 0 : (int64_t)tiles * s * BN * nb * 4;
}

// Accumulate mode needs rows * N fp32 inside the fixed 16 MiB region; larger outputs use ordered mode.
static bool decode_accumulate_ok(int64_t rows, int64_t N) { return rows * N * 4 <= kAccumBytes; }

int64_t decode_workspace_bytes_compact(int64_t rows, int64_t K, int64_t N) {
    const int64_t pb = decode_partial_bytes(rows, K, N);
    return pb ? kCounterBytes + pb : 0;
}

int64_t decode_workspace_bytes(int64_t rows, int64_t K, int64_t N) {
    const int64_t pb = decode_partial_bytes(rows, K, N);
    return pb ? kCounterBytes + kAccumBytes + pb : 0;
}

int64_t decode_workspace_bytes_peer(int64_t rows, int64_t K, int64_t N) { return decode_workspace_bytes(rows, K, N); }

int32_t launch_matmul_decode(const void *a, const void *w, int w_dtype, const void *bias, void *out, int out_dtype,
                             int64_t rows, int64_t K, int64_t N, int act, int flags, void *workspace,
                             int64_t workspace_bytes, bool counters_are_zero, bool compact, cudaStream_t stream,
                             const ttb_peer_gather *gather, const ttb_peer_wait_t *wait) {
    DecodeArgs p = {};
    int tiles, nb;
    decode_plan(rows, K, N, &p.splits, &p.kb_per_split, &tiles, &nb);
    p.w = (const uint8_t *)w; p.a = (const uint16_t *)a; p.bias = (const uint16_t *)bias; p.out = out;
    p.K = K; p.N = N; p.Kt = (int)(K / 32); p.Nt = (int)(N / 32); p.nkb = (int)(K / BK);
    p.act = act; p.out_dtype = out_dtype;
    p.a_row_major = (flags & TTB_MM_A_ROW_MAJOR) != 0;
    p.out_row_major = (flags & TTB_MM_OUT_ROW_MAJOR) != 0;
    p.partial = nullptr; p.accum = nullptr; p.counters = nullptr;
    // Overlap with the previous kernel only when nothing but kernels separates the two launches (no memset below).
    bool overlap = (flags & TTB_MM_WEIGHTS_RESIDENT) != 0;
    p.ordered = compact || (flags & TTB_MM_DETERMINISTIC) != 0 || !decode_accumulate_ok(rows, N);
    p.out_n0 = 0; p.out_N = N; p.out_Nt = p.Nt;
    if (wait) {
        p.wait_arrived = wait->arrived; p.wait_expected = wait->expected;
    }
    if (gather) {
        p.ranks = gather->ranks; p.rank = gather->rank;
        p.out = gather->out[gather->rank];
        p.out_n0 = (int64_t)gather->rank * N; p.out_N = (int64_t)gather->ranks * N; p.out_Nt = gather->ranks * p.Nt;
        for (int r = 0; r < gather->ranks; ++r) {
            p.peer_out[r] = (uint16_t *)gather->out[r];
            p.peer_arrived[r] = gather->arrived[r];
        }
        p.expected = gather->expected;
        p.launch_arrivals = (unsigned)(gather->ranks * tiles);
    }
    if (int32_t rc = status_word_address(&p.status)) return rc;
    if (p.splits > 1) {
        const int64_t need = compact   ? decode_workspace_bytes_compact(rows, K, N)
                             : gather ? decode_workspace_bytes_peer(rows, K, N)
                                      : decode_workspace_bytes(rows, K, N);
        if (!workspace || workspace_bytes < need)
            return fail(TTB_E_WORKSPACE, "ttb_matmul: this shape needs %lld bytes of workspace, got %lld", (long long)need,
                        (long long)workspace_bytes);
        if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
            return fail(TTB_E_INVALID, "ttb_matmul: workspace must be 256-byte aligned");
        p.counters = (int *)workspace;
        p.accum = (float *)((uint8_t *)workspace + kCounterBytes);
        p.partial = (float *)((uint8_t *)workspace + kCounterBytes + (compact ? 0 : kAccumBytes));
        if (!counters_are_zero) {
            // counters always; in accumulate mode also the tiles this launch adds into
            const int64_t zero_bytes = kCounterBytes + (p.ordered ? 0 : rows * N * 4);
            TTB_CUDA_TRY(cudaMemsetAsync(workspace, 0, (size_t)zero_bytes, stream));
            overlap = false;
        }
    }
    dim3 grid((unsigned)(N / BN), (unsigned)p.splits, (unsigned)(rows / nb));
#define TTB_DECODE(F, B) return launch_one<F, B>(p, grid, overlap, stream)
    if (w_dtype == TTB_BFLOAT8_B) {
        // 128 rows per block: the tensor-memory path is the faster one (measured); smaller blocks: the shared-memory path
        // (the gather epilogue and the peer wait exist in the shared-memory kernel only)
        if (!gather && !wait && ((flags & TTB_MM_DECODE_TMEM_OPERAND) || nb == 128)) return launch_decode_tmem(p, nb, grid, overlap, stream);
        if (nb == 32) TTB_DECODE(TTB_BFLOAT8_B, 32);
        if (nb == 64) TTB_DECODE(TTB_BFLOAT8_B, 64);
        TTB_DECODE(TTB_BFLOAT8_B, 128);
    } else {
        if (nb == 32) TTB_DECODE(TTB_BFLOAT4_B, 32);
        if (nb == 64) TTB_DECODE(TTB_BFLOAT4_B, 64);
        TTB_DECODE(TTB_BFLOAT4_B, 128);
    }
#undef TTB_DECODE
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
    if (!decode_supported(w_dtype, rows, K, N))
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
    return decode_workspace_bytes_peer(batch * M, K, N);
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
                                flags & (TTB_MM_A_ROW_MAJOR | TTB_MM_OUT_ROW_MAJOR | TTB_MM_DETERMINISTIC | TTB_MM_WEIGHTS_RESIDENT),
                                workspace, workspace_bytes, (flags & TTB_MM_WORKSPACE_ZEROED) != 0, /*compact=*/false,
                                (cudaStream_t)stream, gather, wait);
}

namespace {
__global__ void peer_wait_kernel(const uint32_t *arrived, const uint32_t *expected_ptr, int *status) {
    const uint32_t expected = *reinterpret_cast<const volatile uint32_t *>(expected_ptr);
    const long long t0 = clock64();
    while ((int)(ttb::ld_acquire_sys(arrived) - expected) < 0) {
        if (clock64() - t0 > 20000000000LL) {
            atomicCAS(status, 0, 7);
            return;
        }
        __nanosleep(100);
    }
}
}  // namespace

extern "C" int32_t ttb_peer_wait(const ttb_peer_wait_t *wait, void *stream) {
    using namespace ttb;
    if (!wait || !wait->arrived || !wait->expected) return fail(TTB_E_INVALID, "ttb_peer_wait: incomplete wait description");
    int *status = nullptr;
    if (int32_t rc = status_word_address(&status)) return rc;
    peer_wait_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(wait->arrived, wait->expected, status);
    TTB_LAUNCH_CHECK("peer_wait");
    return TTB_OK;
}
