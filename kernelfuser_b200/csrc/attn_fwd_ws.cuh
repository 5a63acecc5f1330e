// Warp-specialised, pipelined tcgen05 flash-attention forward kernel (D = 128).
//
// Same operator as attn_fwd_basic.cuh (the reference's `attention_v2_kernel`,
// src/e1_rope_publication_v1.py:609-649, with the Q prologue of :619-623 and the
// rounding contract of `_rows` :551-582), scheduled for the Blackwell tensor
// pipe:
//   * a CTA owns TWO 128-row Q tiles that share one K/V stream - two query
//     heads of the same GQA group at the same query block when the group size
//     is even (identical causal bounds), otherwise two consecutive query
//     blocks of one head;
//   * warps 0-3 / 4-7: softmax + Q prologue + epilogue of tile 0 / tile 1
//     (thread r <-> row r <-> TMEM lane r);  warp 8: TMA producer (K/V rings of
//     128-row tiles, raw Q tiles);  warps 9 / 10: MMA issuer of tile 0 / tile 1
//     (one lane each, chosen by elect.sync so that the MMAs issue on the uniform
//     datapath; the two tiles are independent except for releasing the shared
//     K/V stages);
//   * the KV loop advances in SUB-BLOCKS of 64 keys.  TMEM (512 columns) holds,
//     per tile, two 64-column score buffers and a 128-column output:
//     S0a S0b | S1a S1b | O0 | O1.  Because scores are double-buffered the issuer
//     queues Q K^T of sub-block j+1 BEFORE it waits for the probabilities of
//     sub-block j, so softmax never waits for the tensor pipe and runs
//     back-to-back (throughput-bound, not latency-bound);
//   * P (16-bit) overwrites the score buffer it came from and feeds O += P V as
//     the TMEM A operand; V is an MN-major shared-memory B operand;
//   * the running output is rescaled only when a row's maximum grew by more
//     than 2^8 since the exponent base was last moved (exact after the final
//     division), and only then does softmax wait for the previous P V;
//   * CTAs are ordered (batch, KV head) major, heaviest query block first, so
//     CTAs resident together stream the same K/V through L2.  No cluster
//     multicast anywhere.
// Every wait is bounded and abortable: on expiry the role records a status
// code, raises the CTA's abort flag, and all roles fall through to the common
// exit (bounded wait for copies in flight, TMEM freed).
#pragma once
#include "attn_fwd_basic.cuh"

namespace kf {

enum : int {
    kStatusWsQFull = 201, kStatusWsQReady = 202, kStatusWsKFull = 203, kStatusWsVFull = 204, kStatusWsKEmpty = 205,
    kStatusWsVEmpty = 206, kStatusWsSFull = 207, kStatusWsPReady = 208, kStatusWsODone = 209, kStatusWsPvDone = 210,
};

constexpr int kWsThreads = 352;  // 8 softmax warps, 1 producer warp, 2 issuer warps
constexpr int kWsStages = 2;
constexpr int kWsTileBytes = 2 * kBoxBytes;  // 128 rows x 128 columns of 16-bit values
constexpr int kWsSmemBytes = (2 + 2 * kWsStages) * kWsTileBytes + 1024 + 512;  // tiles, alignment slack, barriers
constexpr int kWsSmemBytesFactored = kWsSmemBytes + 1024;  // + inverse RMS of the Q rows (factored form only)
constexpr float kRescaleThreshold = 8.0f;  // log2 units
constexpr int kSub = 64;                    // keys per sub-block

__device__ __forceinline__ bool mbar_wait_abortable(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 31u) == 0) {
            if (*abort_flag != 0) return false;
            if (clock64() - t0 > kWaitCycles) return false;
        }
    }
}

__device__ __forceinline__ void named_barrier_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Barrier of `nthreads` threads that also returns the OR of their predicates: used to make the outcome of
// per-thread bounded waits uniform across a group before the group meets at further barriers.
__device__ __forceinline__ bool named_barrier_or(int id, int nthreads, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %3, 0;\n\t"
        "bar.red.or.pred p, %1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r)
        : "r"(id), "r"(nthreads), "r"(static_cast<uint32_t>(pred))
        : "memory");
    return r != 0;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// ---- packed fp32 pairs (one instruction for two lanes of the FMA pipe)
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 f2_pack(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(f32x2 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 f2_fma(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 f2_add(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 f2_sub(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

// 2^x for x <= 0 on the FMA pipe (relieves the MUFU unit, which would otherwise
// limit the kernel): n = round(x), f = x - n in [-0.5, 0.5], 2^f by a cubic
// (max relative error 7.5e-5, far below the 16-bit rounding of P), 2^n by an
// integer add into the exponent field.  x is clamped at -125 so the exponent
// never underflows (2^-125 stands in for the 0 of a masked score).
__device__ __forceinline__ void exp2_poly2(float x0, float x1, float& p0, float& p1) {
    const float kMagic = 12582912.f;  // 1.5 * 2^23: adding it rounds to an integer in the low mantissa bits
    x0 = fmaxf(x0, -125.f);
    x1 = fmaxf(x1, -125.f);
    const f32x2 x = f2_pack(x0, x1);
    const f32x2 fr = f2_add(x, f2_pack(kMagic, kMagic));
    const f32x2 f = f2_sub(x, f2_sub(fr, f2_pack(kMagic, kMagic)));
    f32x2 p = f2_fma(f, f2_pack(0.0551716685f, 0.0551716685f), f2_pack(0.2426111251f, 0.2426111251f));
    p = f2_fma(f, p, f2_pack(0.6932609677f, 0.6932609677f));
    p = f2_fma(f, p, f2_pack(0.9999280572f, 0.9999280572f));
    float r0, r1, q0, q1;
    f2_unpack(fr, r0, r1);
    f2_unpack(p, q0, q1);
    p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(r0) << 23));
    p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(r1) << 23));
}

// The polynomial with the score scaling folded in.  The softmax's exponent base m is an
// arbitrary float; the polynomial works from the nearest integer mi = rint(m) (so that
// magic - mi is exact) and its coefficients carry the factor 2^(mi - m), which makes both
// exp paths produce 2^(s*c - m):
//   fr = s*c + (magic - mi)     -> n + magic, n = round(s*c - mi)     (one packed FMA)
//   u  = (magic - mi) - fr      -> -(n + mi), exact
//   f  = s*c + u                -> (s*c - mi) - n in [-0.5, 0.5]      (one packed FMA)
//   p  = 2^(mi - m) * cubic(f) * 2^n
// s is clamped from below at s_min = (mi - 125)/c, which keeps n >= -125 (no exponent
// underflow) and turns a masked -inf score into ~2^-125.
struct PolyBase {
    f32x2 magic_minus_mi, k0, k1, k2, k3;
    float s_min;
    __device__ __forceinline__ void set(float m, float inv_c) {
        const float mi = rintf(m);
        const float k = fast_exp2(mi - m);
        magic_minus_mi = f2_pack(12582912.f - mi, 12582912.f - mi);
        k0 = f2_pack(0.9999280572f * k, 0.9999280572f * k);
        k1 = f2_pack(0.6932609677f * k, 0.6932609677f * k);
        k2 = f2_pack(0.2426111251f * k, 0.2426111251f * k);
        k3 = f2_pack(0.0551716685f * k, 0.0551716685f * k);
        s_min = (mi - 125.f) * inv_c;
    }
};
__device__ __forceinline__ void exp2_poly2_scaled(float s0, float s1, f32x2 c2, const PolyBase& pb, float& p0,
                                                  float& p1) {
    const f32x2 sv = f2_pack(fmaxf(s0, pb.s_min), fmaxf(s1, pb.s_min));
    const f32x2 fr = f2_fma(sv, c2, pb.magic_minus_mi);
    const f32x2 f = f2_fma(sv, c2, f2_sub(pb.magic_minus_mi, fr));
    f32x2 p = f2_fma(f, pb.k3, pb.k2);
    p = f2_fma(f, p, pb.k1);
    p = f2_fma(f, p, pb.k0);
    float r0, r1, q0, q1;
    f2_unpack(fr, r0, r1);
    f2_unpack(p, q0, q1);
    p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(r0) << 23));
    p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(r1) << 23));
}

// Which pairs of a 32-pair sub-block row go through the polynomial (the rest use MUFU ex2).
#ifndef KF_POLY_MASK
#define KF_POLY_MASK 0x88888888u  // every 4th pair: 25 %
#endif
constexpr uint32_t kPolyPairMask = KF_POLY_MASK;

struct WsTile {
    int h, m0, nsub;
};

// FACTORED selects the factored no-RoPE form (raw Q, per-row inverse RMS folded into the softmax scale); it is a
// template parameter so that the standard instantiation carries none of it.
template <typename T, bool FACTORED = false>
__global__ void __launch_bounds__(kWsThreads, 1)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                   const AttnArgs a) {
    constexpr int D = 128;
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kIdescQK = umma_idesc(Num<T>::kFmt, 0, kBM, 64 /* kSub */);
    constexpr uint32_t kIdescPV = umma_idesc(Num<T>::kFmt, 1, kBM, D);

    // An earlier CTA or launch failed: drain quickly.  One thread reads the word and the whole CTA follows that
    // reading, so no warp can leave while others go on to barriers the leaver would have served.
    if (__syncthreads_or(threadIdx.x == 0 && *reinterpret_cast<volatile int*>(a.status) != 0)) return;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_q = smem;                                    // 2 tiles
    uint8_t* smem_k = smem + 2 * kWsTileBytes;                 // kWsStages tiles
    uint8_t* smem_v = smem_k + kWsStages * kWsTileBytes;       // kWsStages tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_v + kWsStages * kWsTileBytes);
    uint64_t* q_full = bars + 0;    // [2] TMA -> softmax group
    uint64_t* q_ready = bars + 2;   // [2] softmax group -> issuer (Q transformed in place)
    uint64_t* k_full = bars + 4;    // [stages]
    uint64_t* k_empty = bars + 6;   // [stages]
    uint64_t* v_full = bars + 8;    // [stages]
    uint64_t* v_empty = bars + 10;  // [stages]
    uint64_t* s_full = bars + 12;   // [tile][buffer] issuer -> softmax group
    uint64_t* p_ready = bars + 16;  // [tile][buffer] softmax group -> issuer (one arrival per warp)
    uint64_t* pv_done = bars + 20;  // [tile][jj & 1] issuer -> softmax group: P V of sub-block jj complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
    volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 25);
    [[maybe_unused]] float* s_inv = reinterpret_cast<float*>(bars + 64);  // [tile][row] inverse RMS of the raw Q rows (factored form)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- work decode
    const int G = a.Hq / a.Hkv;
    const bool pair_heads = (G % 2) == 0;
    const int n_mblk = (a.S + kBM - 1) / kBM;
    const int n_sub_all = (a.S + kSub - 1) / kSub;
    WsTile tile[2];
    int b, kh;
    {
        const int n_mslot = pair_heads ? n_mblk : (n_mblk + 1) / 2;
        const int lanes_per_slot = pair_heads ? G / 2 : G;
        const int upg = n_mslot * lanes_per_slot;  // CTAs per (batch, KV head)
        const int grp = blockIdx.x / upg, r = blockIdx.x % upg;
        b = grp / a.Hkv;
        kh = grp % a.Hkv;
        const int mslot = n_mslot - 1 - r / lanes_per_slot;
        const int sub = r % lanes_per_slot;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            tile[t].h = kh * G + (pair_heads ? 2 * sub + t : sub);
            tile[t].m0 = (pair_heads ? mslot : 2 * mslot + t) * kBM;
            const int full = a.causal ? min((tile[t].m0 + kBM) / kSub, n_sub_all) : n_sub_all;
            tile[t].nsub = (tile[t].m0 < a.S) ? full : 0;
        }
    }
    const int n_sub = max(tile[0].nsub, tile[1].nsub);  // sub-blocks of 64 keys
    const int n_loop = (n_sub + 1) / 2;                 // K/V tiles of 128 keys

    if (tid == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_o);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mbar_init(q_full + i, 1);
            mbar_init(q_ready + i, 4);
            mbar_init(k_full + i, 1);
            mbar_init(k_empty + i, 2);  // one arrival per issuer
            mbar_init(v_full + i, 1);
            mbar_init(v_empty + i, 2);
            mbar_init(s_full + 2 * i, 1);
            mbar_init(s_full + 2 * i + 1, 1);
            mbar_init(p_ready + 2 * i, 4);
            mbar_init(p_ready + 2 * i + 1, 4);
            mbar_init(pv_done + 2 * i, 1);
            mbar_init(pv_done + 2 * i + 1, 1);
        }
        *s_abort = 0;
        fence_mbar_init();
        // The raw Q tiles are requested at once: their trip from DRAM then overlaps the TMEM allocation
        // and the block-wide barrier below instead of following them.
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            if (tile[t].nsub > 0) {
                mbar_expect_tx(q_full + t, kWsTileBytes);
                tma_load_4d(smem_q + t * kWsTileBytes, &tm_q, q_full + t, 0, tile[t].m0, tile[t].h, b);
                tma_load_4d(smem_q + t * kWsTileBytes + kBoxBytes, &tm_q, q_full + t, 64, tile[t].m0, tile[t].h, b);
            }
        }
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    int fail = 0;
    // producer bookkeeping for the exit path (lane 0 of warp 8)
    int k_issued = 0, v_issued = 0;

    if (warp < 8) {
        // =================================================== softmax group t
        const int t = warp >> 2;
        const int r = tid & 127;
        const WsTile tl = (t == 0) ? tile[0] : tile[1];
        if (tl.nsub > 0) {
            uint8_t* my_q = smem_q + t * kWsTileBytes;
            const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
            const uint32_t col_s = t * 128, col_o = 256 + t * 128;
            const int row = tl.m0 + r;
            // ---- Q prologue
            {
                // (all lanes of a warp wait together; the vote keeps them together if the wait runs out)
                auto wait_q = [&]() { return __all_sync(0xffffffffu, mbar_wait_abortable(q_full + t, 0, s_abort)) != 0; };
                bool ok;
                if constexpr (FACTORED) ok = q_inv_coop<D, T>(my_q, r, a, s_inv + t * kBM, wait_q);
                else ok = a.fuse_q ? q_prologue_coop<D, T>(my_q, r, tl.m0, a, wait_q) : wait_q();
                if (!ok) fail = kStatusWsQFull;
            }
            if (!fail) {
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(q_ready + t);
            }
            float m_used = -INFINITY, den = 0.f;
            float c_row = a.scale_log2e;
            if constexpr (FACTORED) {
                // every thread of the group takes part, whatever its wait returned, and all follow the vote
                if (named_barrier_or(1 + t, 128, fail != 0)) { if (!fail) fail = kStatusWsQFull; }
                else c_row *= s_inv[t * kBM + r];
            }
            const float c = c_row;
            bool s_known_ready = false;
            for (int jj = 0; jj < tl.nsub && !fail; ++jj) {
                const int buf = jj & 1;
                const int n0 = jj * kSub;
                const uint32_t col_sb = col_s + buf * kSub;
                // (usually already known from the probe issued during the previous sub-block)
                if (!s_known_ready &&
                    !mbar_wait_abortable(s_full + 2 * t + buf, (jj >> 1) & 1, s_abort)) { fail = kStatusWsSFull; break; }
                tc_fence_after();
                uint32_t sr[2][32];
                tmem_ld32(lane_base + col_sb, sr[0]);
                tmem_ld32(lane_base + col_sb + 32, sr[1]);
                tmem_wait_ld();
                const bool need_mask = (n0 + kSub > a.S) || (a.causal && (n0 + kSub - 1 > tl.m0));
                if (need_mask) {
#pragma unroll
                    for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int n = n0 + q2 * 32 + i;
                            if (n >= a.S || (a.causal && n > row)) sr[q2][i] = 0xff800000u;  // -inf
                        }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        mx0 = max3(mx0, __uint_as_float(sr[q2][i]), __uint_as_float(sr[q2][i + 1]));
                        mx1 = max3(mx1, __uint_as_float(sr[q2][i + 2]), __uint_as_float(sr[q2][i + 3]));
                    }
                const float m_blk = fmaxf(mx0, mx1) * c;
                // move the exponent base only when the maximum grew by more than the threshold
                const bool grow = m_blk > m_used + kRescaleThreshold;
                float alpha = 1.f;
                if (grow) {
                    alpha = fast_exp2(m_used - m_blk);  // 0 on the first sub-block
                    m_used = m_blk;
                    den *= alpha;
                }
                const float neg_m = -m_used;
                const f32x2 c2 = f2_pack(c, c), nm2 = f2_pack(neg_m, neg_m);
                f32x2 psum = f2_pack(0.f, 0.f);
#pragma unroll
                for (int q2 = 0; q2 < 2; ++q2) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float x0, x1, p0, p1;
                        f2_unpack(f2_fma(f2_pack(__uint_as_float(sr[q2][2 * i]), __uint_as_float(sr[q2][2 * i + 1])), c2, nm2),
                                  x0, x1);
                        if ((kPolyPairMask >> (q2 * 16 + i)) & 1u) {
                            exp2_poly2(x0, x1, p0, p1);
                        } else {
                            p0 = fast_exp2(x0);
                            p1 = fast_exp2(x1);
                        }
                        psum = f2_add(psum, f2_pack(p0, p1));
                        pk[i] = Num<T>::pack(p0, p1);
                    }
                    tmem_st16(lane_base + col_sb + q2 * 16, pk);  // P overwrites its S (already in registers)
                }
                // Probe the next score buffer now: the probe is a shared-memory round trip whose latency
                // overlaps the store completion and barrier traffic below.
                s_known_ready = (jj + 1 < tl.nsub) &&
                                mbar_test_wait(s_full + 2 * t + (buf ^ 1), ((jj + 1) >> 1) & 1);
                float ps0, ps1;
                f2_unpack(psum, ps0, ps1);
                den += ps0 + ps1;
                if (jj > 0 && __any_sync(0xffffffffu, grow)) {
                    // O may only be touched once the previous P V has completed.  (pv_done alternates
                    // between two barriers, so a phase cannot be lapped: P V of jj+1 needs this P.)
                    if (!mbar_wait_abortable(pv_done + 2 * t + ((jj - 1) & 1), ((jj - 1) >> 1) & 1, s_abort)) { fail = kStatusWsPvDone; break; }
                    tc_fence_after();
#pragma unroll
                    for (int q4 = 0; q4 < D / 32; ++q4) {
                        uint32_t o[32];
                        tmem_ld32(lane_base + col_o + q4 * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(lane_base + col_o + q4 * 32, o);
                    }
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_ready + 2 * t + buf);
            }
            // ---- epilogue: O / den -> 16-bit -> swizzled smem (this tile's Q buffer) -> TMA store
            if (!fail && !mbar_wait_abortable(pv_done + 2 * t + ((tl.nsub - 1) & 1), ((tl.nsub - 1) >> 1) & 1, s_abort)) fail = kStatusWsODone;
            if (!fail) {
                tc_fence_after();
                const float inv_den = 1.f / den;
                uint8_t* orow = my_q + r * 128;
                const int sw = r & 7;
#pragma unroll
                for (int q4 = 0; q4 < D / 32; ++q4) {
                    uint32_t o[32];
                    tmem_ld32(lane_base + col_o + q4 * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 v4;
                        v4.x = Num<T>::pack(__uint_as_float(o[g * 8 + 0]) * inv_den, __uint_as_float(o[g * 8 + 1]) * inv_den);
                        v4.y = Num<T>::pack(__uint_as_float(o[g * 8 + 2]) * inv_den, __uint_as_float(o[g * 8 + 3]) * inv_den);
                        v4.z = Num<T>::pack(__uint_as_float(o[g * 8 + 4]) * inv_den, __uint_as_float(o[g * 8 + 5]) * inv_den);
                        v4.w = Num<T>::pack(__uint_as_float(o[g * 8 + 6]) * inv_den, __uint_as_float(o[g * 8 + 7]) * inv_den);
                        const int col = q4 * 32 + g * 8;
                        *reinterpret_cast<uint4*>(orow + (col / 64) * kBoxBytes + ((((col % 64) / 8) ^ sw) << 4)) = v4;
                    }
                }
                fence_proxy_async_smem();
            }
            if (fail) {
                *s_abort = 1;
                atomicCAS(a.status, 0, fail);
            }
            tc_fence_before();
            named_barrier_sync(1 + t, 128);
            if ((warp & 3) == 0 && elect_one() && *s_abort == 0) {
                tma_store_4d(&tm_o, my_q, 0, tl.m0, tl.h, b);
                tma_store_4d(&tm_o, my_q + kBoxBytes, 64, tl.m0, tl.h, b);
                tma_store_commit();
                tma_store_wait_read();  // the buffer must outlive the copy's reads; the writes drain on their own
            }
        }
    } else if (warp == 8) {
        // =================================================== TMA producer
        if (elect_one()) {
            for (int j = 0; j < n_loop && !fail; ++j) {
                const int s = j % kWsStages, u = j / kWsStages;
                if (u > 0 && !mbar_wait_abortable(k_empty + s, (u - 1) & 1, s_abort)) { fail = kStatusWsKEmpty; break; }
                mbar_expect_tx(k_full + s, kWsTileBytes);
                tma_load_4d(smem_k + s * kWsTileBytes, &tm_k, k_full + s, 0, j * kBN, kh, b);
                tma_load_4d(smem_k + s * kWsTileBytes + kBoxBytes, &tm_k, k_full + s, 64, j * kBN, kh, b);
                k_issued = j + 1;
                if (u > 0 && !mbar_wait_abortable(v_empty + s, (u - 1) & 1, s_abort)) { fail = kStatusWsVEmpty; break; }
                mbar_expect_tx(v_full + s, kWsTileBytes);
                tma_load_4d(smem_v + s * kWsTileBytes, &tm_v, v_full + s, 0, j * kBN, kh, b);
                tma_load_4d(smem_v + s * kWsTileBytes + kBoxBytes, &tm_v, v_full + s, 64, j * kBN, kh, b);
                v_issued = j + 1;
            }
            if (fail) {
                *s_abort = 1;
                atomicCAS(a.status, 0, fail);
            }
        }
    } else {
        // =================================================== MMA issuer
        if (elect_one()) {
            const uint32_t q_addr = smem_u32(smem_q), k_addr = smem_u32(smem_k), v_addr = smem_u32(smem_v);
            // Descriptors are built once; walking a tile only adds constants to the low word
            // (units of 16 bytes): +2 per 16-column K step inside a 64-column box, +1024 per box,
            // +512 per 64-row half, +2048 per stage, +128 per 16 V rows.
            const uint64_t qk_desc = umma_desc_sw128(0, 16, 1024);        // K-major operands (Q and K)
            const uint64_t v_desc = umma_desc_sw128(0, kBoxBytes, 1024);  // MN-major operand (V)
            const uint32_t qk_hi = static_cast<uint32_t>(qk_desc >> 32), v_hi = static_cast<uint32_t>(v_desc >> 32);
            const uint32_t q_lo = static_cast<uint32_t>(qk_desc) | ((q_addr & 0x3FFFFu) >> 4);
            const uint32_t k_lo = static_cast<uint32_t>(qk_desc) | ((k_addr & 0x3FFFFu) >> 4);
            const uint32_t v_lo = static_cast<uint32_t>(v_desc) | ((v_addr & 0x3FFFFu) >> 4);
            // S_t[buffer jj&1] = Q_t (K rows [64*jj, 64*jj+64))^T
            auto issue_qk = [&](int t, int jj) {
                const uint32_t qa = q_lo + t * (kWsTileBytes >> 4);
                const uint32_t ka = k_lo + ((jj >> 1) % kWsStages) * (kWsTileBytes >> 4) + (jj & 1) * ((kSub * 128) >> 4);
                const uint32_t d = tmem_base + t * 128 + (jj & 1) * kSub;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks / 4) * (kBoxBytes >> 4) + (ks % 4) * 2;
                    umma_ss_lohi(d, qa + off, qk_hi, ka + off, qk_hi, kIdescQK, ks > 0 ? 1u : 0u);
                }
            };
            // O_t += P_t[buffer jj&1] (V rows [64*jj, 64*jj+64))
            auto issue_pv = [&](int t, int jj) {
                const uint32_t va = v_lo + ((jj >> 1) % kWsStages) * (kWsTileBytes >> 4) + (jj & 1) * ((kSub * 128) >> 4);
                const uint32_t d = tmem_base + 256 + t * 128;
                const uint32_t pa = tmem_base + t * 128 + (jj & 1) * kSub;
                umma_ts_lohi(d, pa, va, v_hi, kIdescPV, jj > 0 ? 1u : 0u);
#pragma unroll
                for (int ks = 1; ks < kSub / 16; ++ks) umma_ts_lohi(d, pa + ks * 8, va + ks * 128, v_hi, kIdescPV, 1u);
            };
            const int t = warp - 9;
            const int my_nsub = (t == 0) ? tile[0].nsub : tile[1].nsub;
            // scores of sub-block 0
            if (n_sub > 0 && !mbar_wait_abortable(k_full + 0, 0, s_abort)) fail = kStatusWsKFull;
            if (my_nsub > 0) {
                if (!fail && !mbar_wait_abortable(q_ready + t, 0, s_abort)) fail = kStatusWsQReady;
                if (!fail) {
                    tc_fence_after();
                    issue_qk(t, 0);
                    umma_commit(s_full + 2 * t);
                }
            }
            for (int jj = 0; jj < n_sub && !fail; ++jj) {
                // ---- queue the scores of sub-block jj+1 (their buffer was released by P V of jj-1)
                const int j1 = jj + 1;
                if (j1 < n_sub) {
                    const int st1 = (j1 >> 1) % kWsStages;
                    // (waited for even when this tile has no work left, so that this issuer's
                    // stage releases can never run a whole ring turn ahead of the other issuer's)
                    if ((j1 & 1) == 0 &&
                        !mbar_wait_abortable(k_full + st1, ((j1 >> 1) / kWsStages) & 1, s_abort)) { fail = kStatusWsKFull; break; }
                    if (j1 < my_nsub) {
                        tc_fence_after();
                        issue_qk(t, j1);
                        umma_commit(s_full + 2 * t + (j1 & 1));
                    }
                    if ((j1 & 1) == 1) umma_commit(k_empty + st1);  // this tile is done with both halves of that K tile
                }
                // ---- O += P V of sub-block jj
                const int st0 = (jj >> 1) % kWsStages;
                if ((jj & 1) == 0 &&
                    !mbar_wait_abortable(v_full + st0, ((jj >> 1) / kWsStages) & 1, s_abort)) { fail = kStatusWsVFull; break; }
                if (jj < my_nsub) {
                    if (!mbar_wait_abortable(p_ready + 2 * t + (jj & 1), (jj >> 1) & 1, s_abort)) { fail = kStatusWsPReady; break; }
                    tc_fence_after();
                    issue_pv(t, jj);
                    umma_commit(pv_done + 2 * t + (jj & 1));
                }
                if ((jj & 1) == 1 || jj == n_sub - 1) umma_commit(v_empty + st0);
            }
            if (fail) {
                *s_abort = 1;
                atomicCAS(a.status, 0, fail);
            }
        }
    }

    // ---- common exit
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 8 && *s_abort != 0 && elect_one()) {
        // leave no copy in flight into this CTA's shared memory
#pragma unroll
        for (int t = 0; t < 2; ++t)
            if (tile[t].nsub > 0) mbar_wait(q_full + t, 0);
#pragma unroll
        for (int s = 0; s < kWsStages; ++s) {
            // last load issued into stage s (if any)
            const int lk = ((k_issued - 1 - s) / kWsStages);
            if (k_issued > s) mbar_wait(k_full + s, lk & 1);
            const int lv = ((v_issued - 1 - s) / kWsStages);
            if (v_issued > s) mbar_wait(v_full + s, lv & 1);
        }
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace kf
