// Warp-specialised tcgen05 flash-attention forward kernel (D = 128) that advances in BLOCKS of 128 keys.
//
// Same operator as attn_fwd_ws.cuh (reference: `attention_v2_kernel`,
// src/e1_rope_publication_v1.py:609-649; Q prologue :619-623; rounding contract `_rows` :551-582) and the
// same CTA: two 128-row Q tiles that share one K/V stream, softmax groups of four warps per tile, one TMA
// producer, one MMA issuer per tile.  What differs is the grain of the inner pipeline:
//   * S_t = Q_t K^T is ONE group of N = 128 MMAs per 128-key block (an SS MMA with N = 64 re-reads the
//     4 KB Q slice for half the work and is shared-memory bound); TMEM per tile: 128 score columns and a
//     128-column output;
//   * the softmax thread holds its whole 128-score row in registers: one TMEM load latency, one row
//     maximum, one decision about the exponent base and one round of barrier traffic per 128 keys;
//   * P (16-bit) goes back into the first 64 score columns in four 32-key pieces; the issuer is told after
//     the third piece and again after the fourth, so O += P V starts on the first 96 keys while the last
//     exponentials are still being computed; Q K^T of the next block is queued right behind P V.
// While one tile's softmax runs, the other tile's P V + Q K^T keep the tensor pipe busy.
#pragma once
#include "attn_fwd_ws.cuh"

namespace kf {

enum : int {
    kStatusBkQFull = 401, kStatusBkQReady = 402, kStatusBkKFull = 403, kStatusBkVFull = 404, kStatusBkKEmpty = 405,
    kStatusBkVEmpty = 406, kStatusBkSFull = 407, kStatusBkPReady = 408, kStatusBkODone = 409, kStatusBkPvDone = 410,
};

#ifndef KF_BLK_POLY_MASK
#define KF_BLK_POLY_MASK 0x8888888888888888ull  // pairs of a 64-pair row that go through the polynomial
#endif

// 12 warps: 8 softmax, producer, 2 issuers, 1 spare (so that the last warpgroup is complete for setmaxnreg).
// The CTA starts with 168 registers per thread; the softmax warpgroups take 208 (a 128-score row lives in
// registers), the last warpgroup keeps 88.
constexpr int kBlkThreads = 384;
static_assert(208 * 256 + 88 * 128 <= 65536, "register re-balance");

template <typename T>
__global__ void __launch_bounds__(kBlkThreads, 1)
attn_fwd_blk_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                    const AttnArgs a) {
    constexpr int D = 128;
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kIdescQK = umma_idesc(Num<T>::kFmt, 0, kBM, kBN);
    constexpr uint32_t kIdescPV = umma_idesc(Num<T>::kFmt, 1, kBM, D);
    constexpr unsigned long long kPoly = KF_BLK_POLY_MASK;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_q = smem;                                    // 2 tiles
    uint8_t* smem_k = smem + 2 * kWsTileBytes;                 // kWsStages tiles
    uint8_t* smem_v = smem_k + kWsStages * kWsTileBytes;       // kWsStages tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_v + kWsStages * kWsTileBytes);
    uint64_t* q_full = bars + 0;    // [2] TMA -> softmax group
    uint64_t* q_ready = bars + 2;   // [2] softmax group -> issuer (Q transformed in place)
    uint64_t* k_full = bars + 4;    // [stages]
    uint64_t* k_empty = bars + 6;   // [stages] one arrival per issuer
    uint64_t* v_full = bars + 8;    // [stages]
    uint64_t* v_empty = bars + 10;  // [stages]
    uint64_t* s_full = bars + 12;   // [tile] issuer -> softmax group
    uint64_t* p_a = bars + 14;      // [tile] softmax group -> issuer: P of the block's first 96 keys is in TMEM
    uint64_t* p_b = bars + 16;      // [tile] ... and of the last 32 keys
    uint64_t* pv_done = bars + 18;  // [tile] issuer -> softmax group: P V of the block complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
    volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 21);
    int* s_dead = reinterpret_cast<int*>(bars + 22);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- work decode (as attn_fwd_ws.cuh)
    const int G = a.Hq / a.Hkv;
    const bool pair_heads = (G % 2) == 0;
    const int n_mblk = (a.S + kBM - 1) / kBM;
    const int n_blk_all = (a.S + kBN - 1) / kBN;
    int t_h[2], t_m0[2], t_nblk[2];
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
            t_h[t] = kh * G + (pair_heads ? 2 * sub + t : sub);
            t_m0[t] = (pair_heads ? mslot : 2 * mslot + t) * kBM;
            const int full = a.causal ? min(t_m0[t] / kBN + 1, n_blk_all) : n_blk_all;
            t_nblk[t] = (t_m0[t] < a.S) ? full : 0;
        }
    }
    const int n_blk = max(t_nblk[0], t_nblk[1]);

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
            mbar_init(k_empty + i, 2);
            mbar_init(v_full + i, 1);
            mbar_init(v_empty + i, 2);
            mbar_init(s_full + i, 1);
            mbar_init(p_a + i, 4);
            mbar_init(p_b + i, 4);
            mbar_init(pv_done + i, 1);
        }
        *s_abort = 0;
        *s_dead = *reinterpret_cast<volatile int*>(a.status);  // an earlier CTA failed: the whole CTA drains
        fence_mbar_init();
        if (*s_dead == 0) {
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                if (t_nblk[t] > 0) {
                    mbar_expect_tx(q_full + t, kWsTileBytes);
                    tma_load_4d(smem_q + t * kWsTileBytes, &tm_q, q_full + t, 0, t_m0[t], t_h[t], b);
                    tma_load_4d(smem_q + t * kWsTileBytes + kBoxBytes, &tm_q, q_full + t, 64, t_m0[t], t_h[t], b);
                }
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
    const bool dead = *s_dead != 0;

    int fail = 0;
    int k_issued = 0, v_issued = 0;  // producer bookkeeping for the exit path

    if (dead) {
        // fall through to the common exit
    } else if (warp < 8) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
        // =================================================== softmax group t
        const int t = warp >> 2;
        const int r = tid & 127;
        const int my_nblk = (t == 0) ? t_nblk[0] : t_nblk[1];
        const int my_m0 = (t == 0) ? t_m0[0] : t_m0[1];
        const int my_h = (t == 0) ? t_h[0] : t_h[1];
        if (my_nblk > 0) {
            uint8_t* my_q = smem_q + t * kWsTileBytes;
            const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
            const uint32_t col_s = t * 128, col_o = 256 + t * 128;
            const int row = my_m0 + r;
            // ---- Q prologue
            {
                // (all lanes of a warp wait together; the vote keeps them together if the wait runs out)
                auto wait_q = [&]() { return __all_sync(0xffffffffu, mbar_wait_abortable(q_full + t, 0, s_abort)) != 0; };
                const bool ok = a.fuse_q ? q_prologue_coop<D, T>(my_q, r, my_m0, a, wait_q) : wait_q();
                if (!ok) fail = kStatusBkQFull;
            }
            if (!fail) {
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(q_ready + t);
            }
            float m_used = -INFINITY, den = 0.f;
            const float cs = a.scale_log2e;
            for (int j = 0; j < my_nblk && !fail; ++j) {
                const int n0 = j * kBN;
                if (!mbar_wait_abortable(s_full + t, j & 1, s_abort)) { fail = kStatusBkSFull; break; }
                tc_fence_after();
                uint32_t sr[4][32];
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) tmem_ld32(lane_base + col_s + ch * 32, sr[ch]);
                tmem_wait_ld();
                const bool need_mask = (n0 + kBN > a.S) || (a.causal && (n0 + kBN - 1 > my_m0));
                if (need_mask) {
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch)
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int n = n0 + ch * 32 + i;
                            if (n >= a.S || (a.causal && n > row)) sr[ch][i] = 0xff800000u;  // -inf
                        }
                }
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int ch = 0; ch < 4; ++ch)
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        mx[(i >> 1) & 3] = max3(mx[(i >> 1) & 3], __uint_as_float(sr[ch][i]), __uint_as_float(sr[ch][i + 1]));
                const float m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * cs;
                // move the exponent base only when the maximum grew by more than the threshold
                const bool grow = m_blk > m_used + kRescaleThreshold;
                float alpha = 1.f;
                if (grow) {
                    alpha = fast_exp2(m_used - m_blk);  // 0 on the first block
                    m_used = m_blk;
                    den *= alpha;
                }
                if (j > 0 && __any_sync(0xffffffffu, grow)) {
                    // O may only be touched once the previous P V has completed (it cannot be lapped: P V of
                    // this block needs the probabilities computed below)
                    if (!mbar_wait_abortable(pv_done + t, (j - 1) & 1, s_abort)) { fail = kStatusBkPvDone; break; }
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
                const float neg_m = -m_used;
                const f32x2 c2 = f2_pack(cs, cs), nm2 = f2_pack(neg_m, neg_m);
                f32x2 psum0 = f2_pack(0.f, 0.f), psum1 = f2_pack(0.f, 0.f);
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        float x0, x1, p0, p1;
                        f2_unpack(f2_fma(f2_pack(__uint_as_float(sr[ch][2 * i]), __uint_as_float(sr[ch][2 * i + 1])), c2, nm2),
                                  x0, x1);
                        if ((kPoly >> (ch * 16 + i)) & 1ull) {
                            exp2_poly2(x0, x1, p0, p1);
                        } else {
                            p0 = fast_exp2(x0);
                            p1 = fast_exp2(x1);
                        }
                        if (i & 1) psum1 = f2_add(psum1, f2_pack(p0, p1));
                        else psum0 = f2_add(psum0, f2_pack(p0, p1));
                        pk[i] = Num<T>::pack(p0, p1);
                    }
                    tmem_st16(lane_base + col_s + ch * 16, pk);  // P goes over scores that are already in registers
                    if (ch == 2) {
                        tmem_wait_st();
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(p_a + t);
                    }
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_b + t);
                float ps0, ps1;
                f2_unpack(f2_add(psum0, psum1), ps0, ps1);
                den += ps0 + ps1;
            }
            // ---- epilogue: O / den -> 16-bit -> swizzled smem (this tile's Q buffer) -> TMA store
            if (!fail && !mbar_wait_abortable(pv_done + t, (my_nblk - 1) & 1, s_abort)) fail = kStatusBkODone;
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
            // (every thread of the group gets here, whatever its waits returned)
            const bool bad = named_barrier_or(1 + t, 128, fail != 0);
            if (!bad && (warp & 3) == 0 && elect_one()) {
                tma_store_4d(&tm_o, my_q, 0, my_m0, my_h, b);
                tma_store_4d(&tm_o, my_q + kBoxBytes, 64, my_m0, my_h, b);
                tma_store_commit();
                tma_store_wait_read();  // the buffer must outlive the copy's reads; the writes drain on their own
            }
        }
    } else if (warp == 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
        // =================================================== TMA producer
        if (elect_one()) {
            for (int j = 0; j < n_blk && !fail; ++j) {
                const int s = j % kWsStages, u = j / kWsStages;
                if (u > 0 && !mbar_wait_abortable(k_empty + s, (u - 1) & 1, s_abort)) { fail = kStatusBkKEmpty; break; }
                mbar_expect_tx(k_full + s, kWsTileBytes);
                tma_load_4d(smem_k + s * kWsTileBytes, &tm_k, k_full + s, 0, j * kBN, kh, b);
                tma_load_4d(smem_k + s * kWsTileBytes + kBoxBytes, &tm_k, k_full + s, 64, j * kBN, kh, b);
                k_issued = j + 1;
                if (u > 0 && !mbar_wait_abortable(v_empty + s, (u - 1) & 1, s_abort)) { fail = kStatusBkVEmpty; break; }
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
        asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
        // =================================================== MMA issuer of tile t (warps 9 and 10; warp 11 is spare)
        if (warp < 11 && elect_one()) {
            const int t = warp - 9;
            const int my_nblk = (t == 0) ? t_nblk[0] : t_nblk[1];
            const uint32_t q_addr = smem_u32(smem_q), k_addr = smem_u32(smem_k), v_addr = smem_u32(smem_v);
            const uint64_t qk_desc = umma_desc_sw128(0, 16, 1024);        // K-major operands (Q and K)
            const uint64_t v_desc = umma_desc_sw128(0, kBoxBytes, 1024);  // MN-major operand (V)
            const uint32_t qk_hi = static_cast<uint32_t>(qk_desc >> 32), v_hi = static_cast<uint32_t>(v_desc >> 32);
            const uint32_t q_lo = (static_cast<uint32_t>(qk_desc) | ((q_addr & 0x3FFFFu) >> 4)) + t * (kWsTileBytes >> 4);
            const uint32_t k_lo = static_cast<uint32_t>(qk_desc) | ((k_addr & 0x3FFFFu) >> 4);
            const uint32_t v_lo = static_cast<uint32_t>(v_desc) | ((v_addr & 0x3FFFFu) >> 4);
            const uint32_t d_s = tmem_base + t * 128, d_o = tmem_base + 256 + t * 128;
            // S_t = Q_t (K rows [128*j, 128*j+128))^T
            auto issue_qk = [&](int j) {
                const uint32_t ka = k_lo + (j % kWsStages) * (kWsTileBytes >> 4);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks / 4) * (kBoxBytes >> 4) + (ks % 4) * 2;
                    umma_ss_lohi(d_s, q_lo + off, qk_hi, ka + off, qk_hi, kIdescQK, ks > 0 ? 1u : 0u);
                }
            };
            // O_t += P_t[keys 16*ks0 .. 16*ks1) (V rows of block j)
            auto issue_pv = [&](int j, int ks0, int ks1) {
                const uint32_t va = v_lo + (j % kWsStages) * (kWsTileBytes >> 4);
#pragma unroll
                for (int ks = ks0; ks < ks1; ++ks)
                    umma_ts_lohi(d_o, d_s + ks * 8, va + ks * 128, v_hi, kIdescPV, (j > 0 || ks > 0) ? 1u : 0u);
            };
            if (n_blk > 0 && !mbar_wait_abortable(k_full + 0, 0, s_abort)) fail = kStatusBkKFull;
            if (my_nblk > 0 && !fail) {
                if (!mbar_wait_abortable(q_ready + t, 0, s_abort)) fail = kStatusBkQReady;
                if (!fail) {
                    tc_fence_after();
                    issue_qk(0);
                    umma_commit(s_full + t);
                }
            }
            if (n_blk > 0 && !fail) umma_commit(k_empty + 0);
            for (int j = 0; j < n_blk && !fail; ++j) {
                const int st = j % kWsStages;
                // (stages are waited for and released even when this tile has no work left in them, so that this
                // issuer's releases can never run a whole ring turn ahead of the other issuer's)
                if (!mbar_wait_abortable(v_full + st, (j / kWsStages) & 1, s_abort)) { fail = kStatusBkVFull; break; }
                if (j < my_nblk) {
                    if (!mbar_wait_abortable(p_a + t, j & 1, s_abort)) { fail = kStatusBkPReady; break; }
                    tc_fence_after();
                    issue_pv(j, 0, 6);
                    if (!mbar_wait_abortable(p_b + t, j & 1, s_abort)) { fail = kStatusBkPReady; break; }
                    tc_fence_after();
                    issue_pv(j, 6, 8);
                    umma_commit(pv_done + t);
                }
                umma_commit(v_empty + st);
                if (j + 1 < n_blk) {
                    const int s1 = (j + 1) % kWsStages;
                    if (!mbar_wait_abortable(k_full + s1, ((j + 1) / kWsStages) & 1, s_abort)) { fail = kStatusBkKFull; break; }
                    if (j + 1 < my_nblk) {
                        tc_fence_after();
                        issue_qk(j + 1);
                        umma_commit(s_full + t);
                    }
                    umma_commit(k_empty + s1);
                }
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
    if (!dead && warp == 8 && *s_abort != 0 && elect_one()) {
        // leave no copy in flight into this CTA's shared memory
#pragma unroll
        for (int t = 0; t < 2; ++t)
            if (t_nblk[t] > 0) mbar_wait(q_full + t, 0);
#pragma unroll
        for (int s = 0; s < kWsStages; ++s) {
            if (k_issued > s) mbar_wait(k_full + s, ((k_issued - 1 - s) / kWsStages) & 1);
            if (v_issued > s) mbar_wait(v_full + s, ((v_issued - 1 - s) / kWsStages) & 1);
        }
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace kf
