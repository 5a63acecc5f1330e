// Persistent, warp-specialised tcgen05 flash-attention forward kernel (D = 128).
//
// Same operator and the same inner pipeline as attn_fwd_ws.cuh (reference:
// `attention_v2_kernel`, src/e1_rope_publication_v1.py:609-649; Q prologue
// :619-623; rounding contract `_rows` :551-582).  What changes is the life of a
// CTA: one CTA per SM walks a list of work items (two 128-row Q tiles sharing
// one K/V stream each) and every role keeps running across items, so the
// per-item fixed costs - the raw Q copy, its RMSNorm/RoPE transform, the
// first K/V copies, the output conversion and store - overlap the previous /
// next item's main loop instead of leaving the tensor pipe idle.
//
// Roles (16 warps):
//   warps 0-3 / 4-7   softmax + epilogue of tile 0 / tile 1
//   warp  8           K/V producer (TMA, rings of three 64-row stages each)
//   warps 9 / 10      MMA issuer of tile 0 / tile 1 (one elected lane each)
//   warp  11          Q producer (TMA of raw Q into a double-buffered slot)
//   warps 12-15       Q prologue: RMSNorm + gamma + RoPE in place in shared
//                     memory (no normalised Q ever reaches global memory)
// Shared memory: Q 2 slots x 2 tiles x 32 KB, K 3 x 16 KB, V 3 x 16 KB (224 KB).
// TMEM (512 columns): per tile two 64-column score buffers and a 128-column
// output.  Barrier phases are derived from counters that run across items.
#pragma once
#include "attn_fwd_ws.cuh"

namespace kf {

enum : int {
    kStatusPsQEmpty = 301, kStatusPsQFull = 302, kStatusPsQReady = 303, kStatusPsKFull = 304, kStatusPsVFull = 305,
    kStatusPsKEmpty = 306, kStatusPsVEmpty = 307, kStatusPsSFull = 308, kStatusPsPReady = 309, kStatusPsPvDone = 310,
};

constexpr int kPsThreads = 512;
constexpr int kPsKvStages = 3;
constexpr int kPsKvTileBytes = kSub * 128 * 2;  // 64 rows x 128 columns of 16-bit values (two 8 KB boxes)
constexpr int kPsKvBoxBytes = kSub * 128;       // one 64-column x 64-row box
constexpr int kPsQSlotBytes = 2 * kWsTileBytes; // both tiles of an item
constexpr int kPsSmemBytes = 2 * kPsQSlotBytes + 2 * kPsKvStages * kPsKvTileBytes + 1024 + 512;

struct PsItem {
    int b, kh;
    int h[2], m0[2], nsub[2];
    int n_sub;
};

// Work item `idx` in (batch, KV head)-major order, heaviest query block first
// within a (batch, KV head) group.
__device__ __forceinline__ PsItem ps_decode(int idx, const AttnArgs& a) {
    PsItem it;
    const int G = a.Hq / a.Hkv;
    const bool pair_heads = (G % 2) == 0;
    const int n_mblk = (a.S + kBM - 1) / kBM;
    const int n_sub_all = (a.S + kSub - 1) / kSub;
    const int n_mslot = pair_heads ? n_mblk : (n_mblk + 1) / 2;
    const int lanes_per_slot = pair_heads ? G / 2 : G;
    const int upg = n_mslot * lanes_per_slot;
    const int grp = idx / upg, r = idx % upg;
    it.b = grp / a.Hkv;
    it.kh = grp % a.Hkv;
    const int mslot = n_mslot - 1 - r / lanes_per_slot;
    const int sub = r % lanes_per_slot;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        it.h[t] = it.kh * G + (pair_heads ? 2 * sub + t : sub);
        it.m0[t] = (pair_heads ? mslot : 2 * mslot + t) * kBM;
        const int full = a.causal ? min((it.m0[t] + kBM) / kSub, n_sub_all) : n_sub_all;
        it.nsub[t] = (it.m0[t] < a.S) ? full : 0;
    }
    it.n_sub = max(it.nsub[0], it.nsub[1]);
    return it;
}

#ifdef KF_PROFILE
#define KF_TL(role, n, jj, e) do { if (a.prof != nullptr && blockIdx.x == a.prof_block && (n) == 2 && (jj) >= 16 && (jj) < 24) a.prof[256 + (role) * 128 + ((jj) - 16) * 8 + (e)] = clock64(); } while (0)
#else
#define KF_TL(role, n, jj, e) do {} while (0)
#endif

template <typename T>
__global__ void __launch_bounds__(kPsThreads, 1)
attn_fwd_persist_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                        const AttnArgs a, const int n_items) {
    constexpr int D = 128;
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kIdescQK = umma_idesc(Num<T>::kFmt, 0, kBM, kSub);
    constexpr uint32_t kIdescPV = umma_idesc(Num<T>::kFmt, 1, kBM, D);

    if (*reinterpret_cast<volatile int*>(a.status) != 0) return;  // an earlier launch/CTA failed: drain quickly

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_q = smem;                                          // [slot][tile] 32 KB each
    uint8_t* smem_k = smem + 2 * kPsQSlotBytes;                      // [stage] 16 KB each
    uint8_t* smem_v = smem_k + kPsKvStages * kPsKvTileBytes;         // [stage] 16 KB each
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_v + kPsKvStages * kPsKvTileBytes);
    uint64_t* q_full = bars + 0;     // [slot]   Q producer -> prologue warps
    uint64_t* q_ready = bars + 2;    // [slot]   prologue warps (4 arrivals) -> issuers
    uint64_t* q_empty = bars + 4;    // [slot]   softmax groups (2 arrivals, after the output store read it) -> Q producer
    uint64_t* k_full = bars + 6;     // [stage]
    uint64_t* k_empty = bars + 9;    // [stage]  2 arrivals (one per issuer)
    uint64_t* v_full = bars + 12;    // [stage]
    uint64_t* v_empty = bars + 15;   // [stage]  2 arrivals
    uint64_t* s_full = bars + 18;    // [tile][buffer]
    uint64_t* p_ready = bars + 22;   // [tile][buffer] 4 arrivals (one per softmax warp)
    uint64_t* pv_done = bars + 26;   // [tile][g & 1] issuer -> softmax group: P V of this tile's g-th sub-block complete
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 32);
    volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 33);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_o);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mbar_init(q_full + i, 1);
            mbar_init(q_ready + i, 4);
            mbar_init(q_empty + i, 2);
            mbar_init(s_full + 2 * i, 1);
            mbar_init(s_full + 2 * i + 1, 1);
            mbar_init(p_ready + 2 * i, 4);
            mbar_init(p_ready + 2 * i + 1, 4);
            mbar_init(pv_done + 2 * i, 1);
            mbar_init(pv_done + 2 * i + 1, 1);
        }
#pragma unroll
        for (int i = 0; i < kPsKvStages; ++i) {
            mbar_init(k_full + i, 1);
            mbar_init(k_empty + i, 2);
            mbar_init(v_full + i, 1);
            mbar_init(v_empty + i, 2);
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
    // bookkeeping of the two producers for the exit path
    int kv_issued = 0, q_items_issued = 0;

    // Registers are re-balanced per warpgroup (512 threads start with 128 each): the softmax groups
    // keep a 64-column score row in registers, the other roles need few.
    if (warp < 8) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 176;");
        // ============================================ softmax + epilogue of tile t
        const int t = warp >> 2;
        const int r = tid & 127;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        const uint32_t col_s = t * 128, col_o = 256 + t * 128;
        const float c = a.scale_log2e;
        const float inv_c = 1.f / c;
        int g = 0;  // sub-blocks this tile has processed so far (all items)
        int n = 0;  // items so far
        KF_PROF_DECL;
        for (int idx = blockIdx.x; idx < n_items && !fail; idx += gridDim.x, ++n) {
            const PsItem it = ps_decode(idx, a);
            const int my_nsub = (t == 0) ? it.nsub[0] : it.nsub[1];
            const int my_m0 = (t == 0) ? it.m0[0] : it.m0[1];
            const int my_h = (t == 0) ? it.h[0] : it.h[1];
            const int slot = n & 1;
            if (my_nsub == 0) {
                // Nothing of this tile lives in the slot.  Release it only after this item's Q copy has
                // landed: that copy waited for the slot's previous release, so this group can never
                // deliver two releases into one phase.
                if (r == 0) {
                    if (!mbar_wait_abortable(q_full + slot, (n >> 1) & 1, s_abort)) fail = kStatusPsQFull;
                    else mbar_arrive(q_empty + slot);
                }
                continue;
            }
            uint8_t* my_q = smem_q + slot * kPsQSlotBytes + t * kWsTileBytes;
            const int row = my_m0 + r;
            float m_used = -INFINITY, den = 0.f;
            PolyBase pb;
            pb.set(0.f, inv_c);
            bool s_known_ready = false;
            for (int jj = 0; jj < my_nsub; ++jj) {
                const int gg = g + jj;
                const int buf = gg & 1;
                const int n0 = jj * kSub;
                const uint32_t col_sb = col_s + buf * kSub;
                // (usually already known from the probe issued during the previous sub-block)
                if (!s_known_ready &&
                    !mbar_wait_abortable(s_full + 2 * t + buf, (gg >> 1) & 1, s_abort)) { fail = kStatusPsSFull; break; }
                tc_fence_after();
                KF_PROF(0);
                if ((warp & 3) == 1 && lane == 0) KF_TL(t, n, jj, 0);
                uint32_t sr[2][32];
                tmem_ld32(lane_base + col_sb, sr[0]);
                tmem_ld32(lane_base + col_sb + 32, sr[1]);
                tmem_wait_ld();
                KF_PROF(1);
                const bool need_mask = (n0 + kSub > a.S) || (a.causal && (n0 + kSub - 1 > my_m0));
                if (need_mask) {
#pragma unroll
                    for (int q2 = 0; q2 < 2; ++q2)
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int col = n0 + q2 * 32 + i;
                            if (col >= a.S || (a.causal && col > row)) sr[q2][i] = 0xff800000u;  // -inf
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
                    pb.set(m_used, inv_c);
                }
                const float neg_m = -m_used;
                const f32x2 c2 = f2_pack(c, c), nm2 = f2_pack(neg_m, neg_m);
                f32x2 psum = f2_pack(0.f, 0.f);
                KF_PROF(2);
                if ((warp & 3) == 1 && lane == 0) KF_TL(t, n, jj, 1);
#pragma unroll
                for (int q2 = 0; q2 < 2; ++q2) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float s0 = __uint_as_float(sr[q2][2 * i]), s1 = __uint_as_float(sr[q2][2 * i + 1]);
                        float p0, p1;
                        if ((kPolyPairMask >> (q2 * 16 + i)) & 1u) {
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
                    tmem_st16(lane_base + col_sb + q2 * 16, pk);  // P overwrites its S (already in registers)
                }
                // Probe the next score buffer now: the probe is a shared-memory round trip whose latency
                // overlaps the store completion and barrier traffic below.
                s_known_ready = (jj + 1 < my_nsub) &&
                                mbar_test_wait(s_full + 2 * t + (buf ^ 1), ((gg + 1) >> 1) & 1);
                float ps0, ps1;
                f2_unpack(psum, ps0, ps1);
                den += ps0 + ps1;
                KF_PROF(3);
                if ((warp & 3) == 1 && lane == 0) KF_TL(t, n, jj, 2);
                KF_PROF(4);
                if ((warp & 3) == 1 && lane == 0) KF_TL(t, n, jj, 3);
                if (jj > 0 && __any_sync(0xffffffffu, grow)) {
                    // O may only be touched once the previous P V has completed.  (pv_done alternates
                    // between two barriers, so a phase cannot be lapped: the scores of sub-block g were
                    // written after P V of g-2, the tensor pipe runs in order, and P V of g+1 needs this P.)
                    if (!mbar_wait_abortable(pv_done + 2 * t + ((gg - 1) & 1), ((gg - 1) >> 1) & 1, s_abort)) { fail = kStatusPsPvDone; break; }
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
                KF_PROF(5);
                if ((warp & 3) == 1 && lane == 0) KF_TL(t, n, jj, 4);
            }
            if (fail) break;
            g += my_nsub;
            // ---- epilogue: O / den -> 16-bit -> swizzled smem (this tile's Q slot) -> TMA store
            if (!mbar_wait_abortable(pv_done + 2 * t + ((g - 1) & 1), ((g - 1) >> 1) & 1, s_abort)) { fail = kStatusPsPvDone; break; }
            tc_fence_after();
            {
                const float inv_den = 1.f / den;
                uint8_t* orow = my_q + r * 128;
                const int sw = r & 7;
#pragma unroll
                for (int q4 = 0; q4 < D / 32; ++q4) {
                    uint32_t o[32];
                    tmem_ld32(lane_base + col_o + q4 * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int gq = 0; gq < 4; ++gq) {
                        uint4 v4;
                        v4.x = Num<T>::pack(__uint_as_float(o[gq * 8 + 0]) * inv_den, __uint_as_float(o[gq * 8 + 1]) * inv_den);
                        v4.y = Num<T>::pack(__uint_as_float(o[gq * 8 + 2]) * inv_den, __uint_as_float(o[gq * 8 + 3]) * inv_den);
                        v4.z = Num<T>::pack(__uint_as_float(o[gq * 8 + 4]) * inv_den, __uint_as_float(o[gq * 8 + 5]) * inv_den);
                        v4.w = Num<T>::pack(__uint_as_float(o[gq * 8 + 6]) * inv_den, __uint_as_float(o[gq * 8 + 7]) * inv_den);
                        const int col = q4 * 32 + gq * 8;
                        *reinterpret_cast<uint4*>(orow + (col / 64) * kBoxBytes + ((((col % 64) / 8) ^ sw) << 4)) = v4;
                    }
                }
                fence_proxy_async_smem();
            }
            tc_fence_before();  // the O reads above precede the next item's first P V (ordered through p_ready)
            named_barrier_sync(1 + t, 128);
            if ((warp & 3) == 0 && elect_one()) {
                tma_store_4d(&tm_o, my_q, 0, my_m0, my_h, it.b);
                tma_store_4d(&tm_o, my_q + kBoxBytes, 64, my_m0, my_h, it.b);
                tma_store_commit();
                tma_store_wait_read();  // the slot may be refilled once the copy has read it
                mbar_arrive(q_empty + slot);
            }
            KF_PROF(6);
        }
        if (t == 0 && lane == 0) KF_PROF_FLUSH(warp & 3);
        if (fail) {
            *s_abort = 1;
            atomicCAS(a.status, 0, fail);
        }
        __syncwarp();
        if ((warp & 3) == 0 && elect_one()) tma_store_wait_all();
    } else if (warp < 12) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    if (warp == 8) {
        // ============================================ K/V producer
        if (elect_one()) {
            int gk = 0;  // K/V tiles so far (all items)
            int s = 0;   // ring stage of tile gk
            uint32_t epar = 1;  // parity to wait for on the stage's empty barriers (passes at once on the first turn)
            KF_PROF_DECL;
            for (int idx = blockIdx.x; idx < n_items && !fail; idx += gridDim.x) {
                const PsItem it = ps_decode(idx, a);
                for (int jj = 0; jj < it.n_sub; ++jj, ++gk) {
                    KF_PROF(0);
                    if (!mbar_wait_abortable(k_empty + s, epar, s_abort)) { fail = kStatusPsKEmpty; break; }
                    KF_PROF(1);
                    mbar_expect_tx(k_full + s, kPsKvTileBytes);
                    tma_load_4d(smem_k + s * kPsKvTileBytes, &tm_k, k_full + s, 0, jj * kSub, it.kh, it.b);
                    tma_load_4d(smem_k + s * kPsKvTileBytes + kPsKvBoxBytes, &tm_k, k_full + s, 64, jj * kSub, it.kh, it.b);
                    KF_PROF(2);
                    if (!mbar_wait_abortable(v_empty + s, epar, s_abort)) { fail = kStatusPsVEmpty; break; }
                    KF_PROF(3);
                    mbar_expect_tx(v_full + s, kPsKvTileBytes);
                    tma_load_4d(smem_v + s * kPsKvTileBytes, &tm_v, v_full + s, 0, jj * kSub, it.kh, it.b);
                    tma_load_4d(smem_v + s * kPsKvTileBytes + kPsKvBoxBytes, &tm_v, v_full + s, 64, jj * kSub, it.kh, it.b);
                    kv_issued = gk + 1;
                    KF_PROF(4);
#ifdef KF_PROFILE
                    // latency probe: every 16th tile, wait here for this V tile to land
                    if ((gk & 15) == 15) { mbar_wait(v_full + s, epar ^ 1); KF_PROF(5); }
#endif
                    if (++s == kPsKvStages) { s = 0; epar ^= 1; }
                }
            }
            KF_PROF_FLUSH(4);
            if (fail) {
                *s_abort = 1;
                atomicCAS(a.status, 0, fail);
            }
        }
    } else if (warp == 9 || warp == 10) {
        // ============================================ MMA issuer of tile t
        if (elect_one()) {
            const int t = warp - 9;
            const uint32_t q_addr = smem_u32(smem_q), k_addr = smem_u32(smem_k), v_addr = smem_u32(smem_v);
            // Descriptor low words in units of 16 bytes; walking a tile only adds constants:
            // +2 per 16-column K step inside a 64-column box, +1 box per 64 columns.
            const uint64_t qk_desc = umma_desc_sw128(0, 16, 1024);            // K-major operands (Q and K)
            const uint64_t v_desc = umma_desc_sw128(0, kPsKvBoxBytes, 1024);  // MN-major operand (V), 8 KB between column halves
            const uint32_t qk_hi = static_cast<uint32_t>(qk_desc >> 32), v_hi = static_cast<uint32_t>(v_desc >> 32);
            const uint32_t q_lo = static_cast<uint32_t>(qk_desc) | ((q_addr & 0x3FFFFu) >> 4);
            const uint32_t k_lo = static_cast<uint32_t>(qk_desc) | ((k_addr & 0x3FFFFu) >> 4);
            const uint32_t v_lo = static_cast<uint32_t>(v_desc) | ((v_addr & 0x3FFFFu) >> 4);
            auto issue_qk = [&](uint32_t qa, int stage, int buf) {
                const uint32_t ka = k_lo + stage * (kPsKvTileBytes >> 4);
                const uint32_t d = tmem_base + t * 128 + buf * kSub;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    umma_ss_lohi(d, qa + (ks / 4) * (kBoxBytes >> 4) + (ks % 4) * 2, qk_hi,
                                 ka + (ks / 4) * (kPsKvBoxBytes >> 4) + (ks % 4) * 2, qk_hi, kIdescQK, ks > 0 ? 1u : 0u);
                }
            };
            auto issue_pv = [&](int stage, int buf, uint32_t accumulate) {
                const uint32_t va = v_lo + stage * (kPsKvTileBytes >> 4);
                const uint32_t d = tmem_base + 256 + t * 128;
                const uint32_t pa = tmem_base + t * 128 + buf * kSub;
                umma_ts_lohi(d, pa, va, v_hi, kIdescPV, accumulate);
#pragma unroll
                for (int ks = 1; ks < kSub / 16; ++ks) umma_ts_lohi(d, pa + ks * 8, va + ks * 128, v_hi, kIdescPV, 1u);
            };
            // Running cursors instead of index arithmetic (this single thread's instruction stream is
            // on the critical path): next K tile / V tile to consume, scores and P V issued so far.
            int kst = 0, vst = 0;
            uint32_t kpar = 0, vpar = 0;
            uint32_t nq = 0, np = 0;
            int n = 0;
            KF_PROF_DECL;
            for (int idx = blockIdx.x; idx < n_items && !fail; idx += gridDim.x, ++n) {
                const PsItem it = ps_decode(idx, a);
                const int my_nsub = (t == 0) ? it.nsub[0] : it.nsub[1];
                const int n_sub = it.n_sub;
                const int slot = n & 1;
                const uint32_t qa = q_lo + ((slot * kPsQSlotBytes + t * kWsTileBytes) >> 4);
                if (my_nsub > 0 && !mbar_wait_abortable(q_ready + slot, (n >> 1) & 1, s_abort)) { fail = kStatusPsQReady; break; }
                KF_PROF(0);
                // jq = next sub-block whose scores are to be queued; it runs one ahead of the P V loop.
                // (A K/V stage is waited for and released even when this tile has no work left in it, so
                // that this issuer's releases can never run a whole ring turn ahead of the other issuer's.)
                for (int jj = -1; jj < n_sub; ++jj) {
                    const int jq = jj + 1;
                    if (jq < n_sub) {
                        if (!mbar_wait_abortable(k_full + kst, kpar, s_abort)) { fail = kStatusPsKFull; break; }
                        KF_PROF(1);
                        KF_TL(2 + t, n, jj, 0);
                        if (jq < my_nsub) {
                            tc_fence_after();
                            issue_qk(qa, kst, nq & 1);
                            umma_commit(s_full + 2 * t + (nq & 1));
                            ++nq;
                        }
                        umma_commit(k_empty + kst);
                        if (++kst == kPsKvStages) { kst = 0; kpar ^= 1; }
                        KF_PROF(2);
                        KF_TL(2 + t, n, jj, 1);
                    }
                    if (jj < 0) continue;
                    // ---- O += P V of sub-block jj
                    if (!mbar_wait_abortable(v_full + vst, vpar, s_abort)) { fail = kStatusPsVFull; break; }
                    KF_PROF(3);
                    if (jj < my_nsub) {
                        if (!mbar_wait_abortable(p_ready + 2 * t + (np & 1), (np >> 1) & 1, s_abort)) { fail = kStatusPsPReady; break; }
                        tc_fence_after();
                        KF_PROF(4);
                        KF_TL(2 + t, n, jj, 2);
                        issue_pv(vst, np & 1, jj > 0 ? 1u : 0u);
                        umma_commit(pv_done + 2 * t + (np & 1));
                        ++np;
                    }
                    umma_commit(v_empty + vst);
                    if (++vst == kPsKvStages) { vst = 0; vpar ^= 1; }
                    KF_PROF(5);
                    KF_TL(2 + t, n, jj, 3);
                }
            }
            KF_PROF_FLUSH(5 + t);
            if (fail) {
                *s_abort = 1;
                atomicCAS(a.status, 0, fail);
            }
        }
    } else if (warp == 11) {
        // ============================================ Q producer
        if (elect_one()) {
            int n = 0;
            for (int idx = blockIdx.x; idx < n_items && !fail; idx += gridDim.x, ++n) {
                const PsItem it = ps_decode(idx, a);
                const int slot = n & 1;
                if (n >= 2 && !mbar_wait_abortable(q_empty + slot, ((n >> 1) - 1) & 1, s_abort)) { fail = kStatusPsQEmpty; break; }
                const int active = (it.nsub[0] > 0) + (it.nsub[1] > 0);
                mbar_expect_tx(q_full + slot, active * kWsTileBytes);
#pragma unroll
                for (int t = 0; t < 2; ++t) {
                    if (it.nsub[t] > 0) {
                        uint8_t* dst = smem_q + slot * kPsQSlotBytes + t * kWsTileBytes;
                        tma_load_4d(dst, &tm_q, q_full + slot, 0, it.m0[t], it.h[t], it.b);
                        tma_load_4d(dst + kBoxBytes, &tm_q, q_full + slot, 64, it.m0[t], it.h[t], it.b);
                    }
                }
                q_items_issued = n + 1;
            }
            if (fail) {
                *s_abort = 1;
                atomicCAS(a.status, 0, fail);
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
        // ============================================ Q prologue (warps 12-15)
        const int gtid = tid - 12 * 32;
        int n = 0;
        for (int idx = blockIdx.x; idx < n_items && !fail; idx += gridDim.x, ++n) {
            const PsItem it = ps_decode(idx, a);
            const int slot = n & 1;
            bool waited = false, ok = true;
            auto wait_q = [&]() {
                if (waited) return ok;
                waited = true;
                ok = mbar_wait_abortable(q_full + slot, (n >> 1) & 1, s_abort);
                return ok;
            };
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                if (it.nsub[t] > 0 && a.fuse_q)
                    q_prologue_coop<D, T, 4>(smem_q + slot * kPsQSlotBytes + t * kWsTileBytes, gtid, it.m0[t], a, wait_q);
            }
            if (!wait_q()) { fail = kStatusPsQFull; break; }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_ready + slot);
        }
        if (fail) {
            *s_abort = 1;
            atomicCAS(a.status, 0, fail);
        }
    }

    // ---- common exit
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (*s_abort != 0) {
        // leave no copy in flight into this CTA's shared memory
        if (warp == 8 && elect_one()) {
#pragma unroll
            for (int s = 0; s < kPsKvStages; ++s) {
                if (kv_issued > s) {
                    const int last_u = (kv_issued - 1 - s) / kPsKvStages;
                    mbar_wait(k_full + s, last_u & 1);
                    mbar_wait(v_full + s, last_u & 1);
                }
            }
        }
        if (warp == 11 && elect_one()) {
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                if (q_items_issued > s) mbar_wait(q_full + s, ((q_items_issued - 1 - s) / 2) & 1);
            }
        }
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace kf
