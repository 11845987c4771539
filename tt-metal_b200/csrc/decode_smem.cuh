// Constants, shared-memory layout and the exact packed -> bf16 expansion shared by the shared-memory-operand decode kernels.
#pragma once
#include <type_traits>

#include "decode_common.cuh"

namespace ttb {
namespace decode_smem {

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

}  // namespace decode_smem
}  // namespace ttb
