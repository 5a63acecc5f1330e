// Row-prepare kernel: y[b,h,s,:] = RoPE(RMSNorm(x[b,h,s,:]) * gamma), position = s.
//
// Replaces the reference's `prepare_kernel` (src/e1_rope_publication_v1.py:586-605,
// launched by `prepare_attention` :652-658) for K (and for Q in the unfused
// mode).  Pure HBM streaming: algorithmic traffic is one read of x and one
// write of y (2 * rows * D * 2 bytes).
//
// Mapping.  A row of D 16-bit values is covered by D/16 lanes; each lane owns
// the 16-byte chunk at columns [8i, 8i+8) and its rotation partner at
// [D/2+8i, D/2+8i+8), so the split-half rotation needs no shuffle and the
// sum of squares needs log2(D/16) xor-shuffles.  A CTA owns a range of
// POSITIONS and walks over (batch, head) pairs: the cos/sin chunks of a
// position are loaded once into registers and reused for every pair, so
// the tables are read once per CTA instead of once per row.  Two rows are in
// flight per lane and the register budget is held to 64 so that four CTAs
// (32 warps) share an SM: measured on B200 that is the best trade between
// loads in flight per lane and resident warps (80 % / 86 % of the measured
// copy bandwidth at D = 128 / 256).
#pragma once
#include "rounding.cuh"

namespace kf {

struct PrepareArgs {
    const void* x;
    void* y;
    const void* gamma;  // [D]
    const void* gamma2; // [D] second weight vector of the factored no-RoPE form, else null
    const void* cos;    // [S, D] or null
    const void* sin;    // [S, D] or null
    long long x_sb, x_sh, x_ss;  // element strides of x (batch, head, row); D is contiguous
    long long y_sb, y_sh, y_ss;
    int B, H, S;
    int bh_per_cta;  // (batch, head) pairs per CTA along grid.y
    float eps;
    int rope, hf_norm;
};

#ifndef KF_PREP_UNROLL
#define KF_PREP_UNROLL 2
#endif
#ifndef KF_PREP_MINBLK
#define KF_PREP_MINBLK 4
#endif
constexpr int kPrepThreads = 256;
constexpr int kPrepUnroll = KF_PREP_UNROLL;  // rows in flight per lane

// FACTORED: y = r(x * inv * gamma * gamma2), one rounding, no rotation - the K side of the reference's
// factored no-RoPE form (`prepare_factored_kernel`, src/e1_qk_publication_v3.py:593-611), which folds the
// query weight into the prepared keys so that the query itself needs only its inverse RMS.
template <int D, typename T, bool FACTORED = false>
__global__ void __launch_bounds__(kPrepThreads, KF_PREP_MINBLK) prepare_rows_kernel(const PrepareArgs a) {
    constexpr int LPR = D / 16;                      // lanes per row
    constexpr int RPW = 32 / LPR;                    // rows per warp
    constexpr int RPB = RPW * (kPrepThreads / 32);   // positions per CTA
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // an attention kernel launched as a programmatic dependent may start its own prologue now; it reads the
    // rows written here only after its griddepcontrol.wait
    grid_dep_launch_dependents();
    const int sub = lane % LPR;                      // chunk index within the half row
    const int pos = blockIdx.x * RPB + warp * RPW + lane / LPR;
    const bool valid = pos < a.S;
    const bool rope = a.rope != 0, hf = a.hf_norm != 0;

    const uint4* g4 = reinterpret_cast<const uint4*>(a.gamma);
    const uint4 glo = __ldg(g4 + sub), ghi = __ldg(g4 + LPR + sub);
    uint4 clo = make_uint4(0, 0, 0, 0), chi = clo, slo = clo, shi = clo;
    if constexpr (FACTORED) {  // the table registers carry the second weight vector instead
        const uint4* h4 = reinterpret_cast<const uint4*>(a.gamma2);
        clo = __ldg(h4 + sub);
        chi = __ldg(h4 + LPR + sub);
    } else if (rope && valid) {
        const uint4* c4 = reinterpret_cast<const uint4*>(a.cos) + static_cast<long long>(pos) * (D / 8);
        const uint4* s4 = reinterpret_cast<const uint4*>(a.sin) + static_cast<long long>(pos) * (D / 8);
        clo = __ldg(c4 + sub);
        chi = __ldg(c4 + LPR + sub);
        slo = __ldg(s4 + sub);
        shi = __ldg(s4 + LPR + sub);
    }

    const int BH = a.B * a.H;
    const int bh0 = blockIdx.y * a.bh_per_cta;
    const int bh1 = min(bh0 + a.bh_per_cta, BH);
    const T* xb = reinterpret_cast<const T*>(a.x);
    T* yb = reinterpret_cast<T*>(a.y);

    for (int bh = bh0; bh < bh1; bh += kPrepUnroll) {
        uint4 lo[kPrepUnroll], hi[kPrepUnroll];
#pragma unroll
        for (int u = 0; u < kPrepUnroll; ++u) {
            const int p = bh + u;
            if (valid && p < bh1) {
                const int b = p / a.H, h = p - b * a.H;
                const uint4* src = reinterpret_cast<const uint4*>(xb + b * a.x_sb + h * a.x_sh + pos * a.x_ss);
                lo[u] = __ldcs(src + sub);
                hi[u] = __ldcs(src + LPR + sub);
            } else {
                lo[u] = make_uint4(0, 0, 0, 0);
                hi[u] = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int u = 0; u < kPrepUnroll; ++u) {
            const int p = bh + u;
            float ss = sumsq_chunk<T>(hi[u], sumsq_chunk<T>(lo[u], 0.f));
#pragma unroll
            for (int m = LPR / 2; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
            const float inv = rsqrtf(ss * (1.0f / static_cast<float>(D)) + a.eps);
            if constexpr (FACTORED) {
                scale_chunk2<T>(lo[u], inv, glo, clo);
                scale_chunk2<T>(hi[u], inv, ghi, chi);
            } else {
                transform_pair<T>(lo[u], hi[u], inv, glo, ghi, clo, chi, slo, shi, hf, rope);
            }
            if (valid && p < bh1) {
                const int b = p / a.H, h = p - b * a.H;
                uint4* dst = reinterpret_cast<uint4*>(yb + b * a.y_sb + h * a.y_sh + pos * a.y_ss);
                dst[sub] = lo[u];
                dst[LPR + sub] = hi[u];
            }
        }
    }
}

}  // namespace kf
