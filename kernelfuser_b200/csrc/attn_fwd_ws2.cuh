// Pipelined tcgen05 flash-attention forward kernel (D = 128) with TWO warps per group of 32 rows.
//
// Same operator, work decomposition, TMEM/shared-memory layout, producer and MMA-issuer roles as
// attn_fwd_ws.cuh (reference: `attention_v2_kernel`, src/e1_rope_publication_v1.py:609-649, Q
// prologue :619-623, rounding contract `_rows` :551-582).  The softmax of a 64-key sub-block is
// split by columns between two warps that own the same 32 TMEM lanes (rows): each loads 32
// score columns, they agree on the row maximum through shared memory, and each computes its 32
// exponentials, its partial denominator and its half of P; the 128 output columns are split the
// same way for the rare rescale and for the epilogue.  With four softmax warps per scheduler
// instead of two, the TMEM load / store latencies, the max reduction and the barrier traffic of
// one warp overlap the MUFU-bound exponentials of another, which is what limits the
// one-thread-per-row layout.
//
// Warps: 0-7 tile 0 (0-3 columns [0,32), 4-7 columns [32,64)), 8-15 tile 1, 16 TMA producer,
// 17 / 18 MMA issuers, 19 spare.
#pragma once
#include "attn_fwd_ws.cuh"

namespace kf {

constexpr int kWs2Threads = 640;
constexpr int kWs2SmemBytes = kWsSmemBytes + 4096;
constexpr int kStatusWsXchg = 211;

template <typename T>
__global__ void __launch_bounds__(kWs2Threads, 1)
attn_fwd_ws2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                   const AttnArgs a) {
    constexpr int D = 128;
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kIdescQK = umma_idesc(Num<T>::kFmt, 0, kBM, 64 /* kSub */);
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
    uint64_t* s_full = bars + 12;   // [tile][buffer] issuer -> softmax group
    uint64_t* p_ready = bars + 16;  // [tile][buffer] softmax group -> issuer (one arrival per warp)
    uint64_t* pv_done = bars + 20;  // [tile] issuer -> softmax group, one phase per sub-block
    uint64_t* x_bar = bars + 24;    // [tile][row quarter] max / denominator exchange between the two column halves
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 32);
    volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 33);
    float* xchg = reinterpret_cast<float*>(bars + 40);  // [tile][half][parity][row]

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
            mbar_init(p_ready + 2 * i, 8);      // one arrival per softmax warp of the tile
            mbar_init(p_ready + 2 * i + 1, 8);
            mbar_init(pv_done + i, 1);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) mbar_init(x_bar + i, 2);
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

    if (warp < 16) {
        // =================================================== softmax: tile t, column half `half`, rows r
        // Two warps share each group of 32 rows: one owns columns [0,32) of every 64-key sub-block,
        // the other columns [32,64).  They agree on the row maximum through shared memory and an
        // mbarrier per (tile, row quarter); everything else (exponentials, partial denominators,
        // P stores, half of the O columns) is private to a warp.
        const int t = warp >> 3;
        const int half = (warp >> 2) & 1;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const WsTile tl = (t == 0) ? tile[0] : tile[1];
        if (tl.nsub > 0) {
            uint8_t* my_q = smem_q + t * kWsTileBytes;
            const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
            const uint32_t col_s = t * 128, col_o = 256 + t * 128 + half * 64;
            const int row = tl.m0 + r;
            uint64_t* xbar = x_bar + t * 4 + quarter;
            float* my_x = xchg + (t * 2 + half) * 256 + r;          // [tile][half][parity][row]
            const float* peer_x = xchg + (t * 2 + (half ^ 1)) * 256 + r;
            // ---- Q prologue (the column-half-0 warps transform the tile; the others only wait)
            if (half == 0) {
                auto wait_q = [&]() { return mbar_wait_abortable(q_full + t, 0, s_abort); };
                const bool ok = a.fuse_q ? q_prologue_coop<D, T, 4>(my_q, r, tl.m0, a, wait_q) : wait_q();
                if (!ok) fail = kStatusWsQFull;
                if (!fail) {
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(q_ready + t);
                }
            }
            float m_used = -INFINITY, den = 0.f;
            const float c = a.scale_log2e;
            const float inv_c = 1.f / c;
            PolyBase pb;
            pb.set(0.f, inv_c);
            for (int jj = 0; jj < tl.nsub && !fail; ++jj) {
                const int buf = jj & 1;
                const int n0 = jj * kSub + half * 32;
                const uint32_t col_sb = col_s + buf * kSub;
                if (!mbar_wait_abortable(s_full + 2 * t + buf, (jj >> 1) & 1, s_abort)) { fail = kStatusWsSFull; break; }
                tc_fence_after();
                uint32_t sr[32];
                tmem_ld32(lane_base + col_sb + half * 32, sr);
                tmem_wait_ld();
                const bool need_mask = (n0 + 32 > a.S) || (a.causal && (n0 + 31 > tl.m0));
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int n = n0 + i;
                        if (n >= a.S || (a.causal && n > row)) sr[i] = 0xff800000u;  // -inf
                    }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    mx0 = max3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
                    mx1 = max3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
                }
                const float mx_mine = fmaxf(mx0, mx1);
                // ---- agree on the row maximum with the warp that owns the other 32 columns
                my_x[buf * 128] = mx_mine;
                __syncwarp();
                if (lane == 0) mbar_arrive(xbar);
                if (!mbar_wait_abortable(xbar, jj & 1, s_abort)) { fail = kStatusWsXchg; break; }
                const float m_blk = fmaxf(mx_mine, peer_x[buf * 128]) * c;
                // (past this point the peer has finished reading its scores, so P may overwrite them)
                // move the exponent base only when the maximum grew by more than the threshold
                const bool grow = m_blk > m_used + kRescaleThreshold;
                float alpha = 1.f;
                if (grow) {
                    alpha = fast_exp2(m_used - m_blk);  // 0 on the first sub-block
                    m_used = m_blk;
                    den *= alpha;
                    pb.set(m_used, inv_c);
                }
                const float neg_m = -m_used;
                const f32x2 c2 = f2_pack(c, c), nm2 = f2_pack(neg_m, neg_m);
                f32x2 psum = f2_pack(0.f, 0.f);
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float s0 = __uint_as_float(sr[2 * i]), s1 = __uint_as_float(sr[2 * i + 1]);
                    float p0, p1;
                    if ((kPolyPairMask >> i) & 1u) {
                        exp2_poly2_scaled(s0, s1, c2, pb, p0, p1);
                    } else {
                        float x0, x1;
                        f2_unpack(f2_fma(f2_pack(s0, s1), c2, nm2), x0, x1);
                        p0 = fast_exp2(x0);
                        p1 = fast_exp2(x1);
                    }
                    psum = f2_add(psum, f2_pack(p0, p1));
                    pk[i] = Num<T>::pack(p0, p1);
                }
                tmem_st16(lane_base + col_sb + half * 16, pk);  // P (16-bit) overwrites the score buffer
                float ps0, ps1;
                f2_unpack(psum, ps0, ps1);
                den += ps0 + ps1;
                // Track the completion of the previous P V every sub-block (normally long past):
                // it keeps this warp within one phase of pv_done, and O may only be touched
                // after it.
                if (jj > 0 && !mbar_wait_abortable(pv_done + t, (jj - 1) & 1, s_abort)) { fail = kStatusWsPvDone; break; }
                if (jj > 0 && __any_sync(0xffffffffu, grow)) {  // this warp rescales its 64 O columns
                    tc_fence_after();
#pragma unroll
                    for (int q4 = 0; q4 < 2; ++q4) {
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
            // ---- total denominator: add the other warp's partial sum
            if (!fail) {
                const int pb2 = tl.nsub & 1;
                my_x[pb2 * 128] = den;
                __syncwarp();
                if (lane == 0) mbar_arrive(xbar);
                if (!mbar_wait_abortable(xbar, tl.nsub & 1, s_abort)) fail = kStatusWsXchg;
                else den += peer_x[pb2 * 128];
            }
            // ---- epilogue: this warp's 64 O columns / den -> 16-bit -> swizzled smem (the tile's Q buffer)
            if (!fail && !mbar_wait_abortable(pv_done + t, (tl.nsub - 1) & 1, s_abort)) fail = kStatusWsODone;
            if (!fail) {
                tc_fence_after();
                const float inv_den = 1.f / den;
                uint8_t* orow = my_q + half * kBoxBytes + r * 128;
                const int sw = r & 7;
#pragma unroll
                for (int q4 = 0; q4 < 2; ++q4) {
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
                        const int ch = q4 * 4 + g;  // 16-byte chunk within this warp's 64-column box
                        *reinterpret_cast<uint4*>(orow + ((ch ^ sw) << 4)) = v4;
                    }
                }
                fence_proxy_async_smem();
            }
            if (fail) {
                *s_abort = 1;
                atomicCAS(a.status, 0, fail);
            }
            tc_fence_before();
            named_barrier_sync(1 + t, 256);
            if (half == 0 && quarter == 0 && elect_one() && *s_abort == 0) {
                tma_store_4d(&tm_o, my_q, 0, tl.m0, tl.h, b);
                tma_store_4d(&tm_o, my_q + kBoxBytes, 64, tl.m0, tl.h, b);
                tma_store_commit();
                tma_store_wait_read();  // the buffer must outlive the copy's reads; the writes drain on their own
            }
        }
    } else if (warp == 16) {
        // =================================================== TMA producer
        if (elect_one()) {
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                if (tile[t].nsub > 0) {
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
    } else if (warp < 19) {
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
            const int t = warp - 17;
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
                    umma_commit(pv_done + t);
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
    if (warp == 16 && *s_abort != 0 && elect_one()) {
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
