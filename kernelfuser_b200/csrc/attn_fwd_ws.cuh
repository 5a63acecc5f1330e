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
//     two stages each, raw Q tiles);  warp 9: MMA issuer (one elected lane);
//   * TMEM (512 columns): S0 | S1 | O0 | O1, 128 fp32 columns each; P (16-bit)
//     overwrites its S and feeds O += P V as the TMEM A operand;
//   * the issuer alternates tiles: PV0(j), QK0(j+1), PV1(j), QK1(j+1) - while
//     one tile's rows are in softmax the tensor pipe works for the other;
//   * the running output is rescaled only when a row's maximum grew by more
//     than 2^8 since the exponent base was last moved (exact after the final
//     division; keeps tcgen05.ld/st of O off the critical path);
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
    kStatusWsVEmpty = 206, kStatusWsSFull = 207, kStatusWsPReady = 208, kStatusWsODone = 209,
};

constexpr int kWsThreads = 320;
constexpr int kWsStages = 2;
constexpr int kWsTileBytes = 2 * kBoxBytes;  // 128 rows x 128 columns of 16-bit values
constexpr int kWsSmemBytes = (2 + 2 * kWsStages) * kWsTileBytes + 1024 + 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

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

__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

struct WsTile {
    int h, m0, nblk;
};

template <typename T>
__global__ void __launch_bounds__(kWsThreads, 1)
attn_fwd_ws_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                   const AttnArgs a) {
    constexpr int D = 128;
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kIdescQK = umma_idesc(Num<T>::kFmt, 0, kBM, kBN);
    constexpr uint32_t kIdescPV = umma_idesc(Num<T>::kFmt, 1, kBM, D);

    if (*reinterpret_cast<volatile int*>(a.status) != 0) return;  // an earlier CTA failed: drain quickly

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
    uint64_t* s_full = bars + 12;   // [2] issuer -> softmax group
    uint64_t* p_ready = bars + 14;  // [2] softmax group -> issuer
    uint64_t* o_done = bars + 16;   // [2] issuer -> softmax group (last PV complete)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
    volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 25);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- work decode
    const int G = a.Hq / a.Hkv;
    const bool pair_heads = (G % 2) == 0;
    const int n_mblk = (a.S + kBM - 1) / kBM;
    const int n_kv_all = (a.S + kBN - 1) / kBN;
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
            const int full = a.causal ? min((tile[t].m0 + kBM + kBN - 1) / kBN, n_kv_all) : n_kv_all;
            tile[t].nblk = (tile[t].m0 < a.S) ? full : 0;
        }
    }
    const int n_loop = max(tile[0].nblk, tile[1].nblk);

    if (tid == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_o);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mbar_init(q_full + i, 1);
            mbar_init(q_ready + i, 128);
            mbar_init(k_full + i, 1);
            mbar_init(k_empty + i, 1);
            mbar_init(v_full + i, 1);
            mbar_init(v_empty + i, 1);
            mbar_init(s_full + i, 1);
            mbar_init(p_ready + i, 128);
            mbar_init(o_done + i, 1);
        }
        *s_abort = 0;
        fence_mbar_init();
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
    int k_issued = 0, v_issued = 0, q_issued[2] = {0, 0};

    if (warp < 8) {
        // =================================================== softmax group t
        const int t = warp >> 2;
        const int r = tid & 127;
        const WsTile tl = (t == 0) ? tile[0] : tile[1];
        if (tl.nblk > 0) {
            uint8_t* my_q = smem_q + t * kWsTileBytes;
            const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
            const uint32_t col_s = t * 128, col_o = 256 + t * 128;
            const int row = tl.m0 + r;
            // ---- Q prologue
            if (!mbar_wait_abortable(q_full + t, 0, s_abort)) fail = kStatusWsQFull;
            if (!fail) {
                if (a.fuse_q) q_prologue_inplace<D, T>(my_q, r, row, a);
                fence_proxy_async_smem();
                mbar_arrive(q_ready + t);
            }
            float m_used = -INFINITY, den = 0.f;
            const float c = a.scale_log2e;
            for (int j = 0; j < tl.nblk && !fail; ++j) {
                const int n0 = j * kBN;
                if (!mbar_wait_abortable(s_full + t, j & 1, s_abort)) { fail = kStatusWsSFull; break; }
                tc_fence_after();
                uint32_t sr[4][32];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) tmem_ld32(lane_base + col_s + q4 * 32, sr[q4]);
                tmem_wait_ld();
                const bool need_mask = (n0 + kBN > a.S) || (a.causal && (n0 + kBN - 1 > tl.m0));
                if (need_mask) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int n = n0 + q4 * 32 + i;
                            if (n >= a.S || (a.causal && n > row)) sr[q4][i] = 0xff800000u;  // -inf
                        }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        mx0 = max3(mx0, __uint_as_float(sr[q4][i]), __uint_as_float(sr[q4][i + 1]));
                        mx1 = max3(mx1, __uint_as_float(sr[q4][i + 2]), __uint_as_float(sr[q4][i + 3]));
                    }
                const float m_blk = fmaxf(mx0, mx1) * c;
                // move the exponent base only when the maximum grew by more than the threshold
                const bool grow = m_blk > m_used + kRescaleThreshold;
                float alpha = 1.f;
                if (grow) {
                    alpha = fast_exp2(m_used - m_blk);  // 0 on the first block
                    m_used = m_blk;
                    den *= alpha;
                }
                const float neg_m = -m_used;
                float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float p0 = fast_exp2(fmaf(__uint_as_float(sr[q4][2 * i]), c, neg_m));
                        const float p1 = fast_exp2(fmaf(__uint_as_float(sr[q4][2 * i + 1]), c, neg_m));
                        ps0 += p0;
                        ps1 += p1;
                        pk[i] = Num<T>::pack(p0, p1);
                    }
                    tmem_st16(lane_base + col_s + q4 * 16, pk);  // P overwrites S (already in registers)
                }
                den += ps0 + ps1;
                // S(j) complete implies PV(j-1) complete, so O may be touched here
                if (j > 0 && __any_sync(0xffffffffu, grow)) {
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
                mbar_arrive(p_ready + t);
            }
            // ---- epilogue: O / den -> 16-bit -> swizzled smem (this tile's Q buffer) -> TMA store
            if (!fail && !mbar_wait_abortable(o_done + t, 0, s_abort)) fail = kStatusWsODone;
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
            if (r == 0 && *s_abort == 0) {
                tma_store_4d(&tm_o, my_q, 0, tl.m0, tl.h, b);
                tma_store_4d(&tm_o, my_q + kBoxBytes, 64, tl.m0, tl.h, b);
                tma_store_commit();
                tma_store_wait_all();
            }
        }
    } else if (warp == 8) {
        // =================================================== TMA producer
        if (lane == 0) {
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                if (tile[t].nblk > 0) {
                    mbar_expect_tx(q_full + t, kWsTileBytes);
                    tma_load_4d(smem_q + t * kWsTileBytes, &tm_q, q_full + t, 0, tile[t].m0, tile[t].h, b);
                    tma_load_4d(smem_q + t * kWsTileBytes + kBoxBytes, &tm_q, q_full + t, 64, tile[t].m0, tile[t].h, b);
                    q_issued[t] = 1;
                }
            }
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
        if (lane == 0) {
            const uint32_t q_addr = smem_u32(smem_q), k_addr = smem_u32(smem_k), v_addr = smem_u32(smem_v);
            auto issue_qk = [&](int t, int stage) {
                const uint32_t qa = q_addr + t * kWsTileBytes, ka = k_addr + stage * kWsTileBytes;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks / 4) * kBoxBytes + (ks % 4) * 32;
                    umma_ss(tmem_base + t * 128, umma_desc_sw128(qa + off, 16, 1024), umma_desc_sw128(ka + off, 16, 1024),
                            kIdescQK, ks > 0);
                }
            };
            auto issue_pv = [&](int t, int stage, bool accumulate) {
                const uint32_t va = v_addr + stage * kWsTileBytes;
#pragma unroll
                for (int ks = 0; ks < kBN / 16; ++ks) {
                    umma_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + ks * 8,
                            umma_desc_sw128(va + ks * 2048, kBoxBytes, 1024), kIdescPV, accumulate || ks > 0);
                }
            };
            // block 0 scores
            if (n_loop > 0) {
                if (!mbar_wait_abortable(k_full + 0, 0, s_abort)) fail = kStatusWsKFull;
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (!fail && tile[t].nblk > 0) {
                        if (!mbar_wait_abortable(q_ready + t, 0, s_abort)) { fail = kStatusWsQReady; break; }
                        tc_fence_after();
                        issue_qk(t, 0);
                        umma_commit(s_full + t);
                    }
                }
                if (!fail) umma_commit(k_empty + 0);
            }
            for (int j = 0; j < n_loop && !fail; ++j) {
                const int sv = j % kWsStages;
                const int sk1 = (j + 1) % kWsStages;
                if (!mbar_wait_abortable(v_full + sv, (j / kWsStages) & 1, s_abort)) { fail = kStatusWsVFull; break; }
                if (j + 1 < n_loop &&
                    !mbar_wait_abortable(k_full + sk1, ((j + 1) / kWsStages) & 1, s_abort)) { fail = kStatusWsKFull; break; }
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (j < tile[t].nblk) {
                        if (!mbar_wait_abortable(p_ready + t, j & 1, s_abort)) { fail = kStatusWsPReady; break; }
                        tc_fence_after();
                        issue_pv(t, sv, j > 0);
                        if (j + 1 < tile[t].nblk) {
                            issue_qk(t, sk1);
                            umma_commit(s_full + t);
                        } else {
                            umma_commit(o_done + t);
                        }
                    }
                }
                if (fail) break;
                umma_commit(v_empty + sv);
                if (j + 1 < n_loop) umma_commit(k_empty + sk1);
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
    if (warp == 8 && lane == 0 && *s_abort != 0) {
        // leave no copy in flight into this CTA's shared memory
#pragma unroll
        for (int t = 0; t < 2; ++t)
            if (q_issued[t]) mbar_wait(q_full + t, 0);
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
