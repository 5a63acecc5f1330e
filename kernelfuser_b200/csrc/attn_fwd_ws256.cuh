// Warp-specialised, pipelined tcgen05 flash-attention forward kernel with ONE 128-row Q tile per CTA
// (all of D = 256; D = 128 for launches of moderate size, two CTAs per SM).
//
// Same operator as the other attention kernels (reference: `attention_v2_kernel`,
// src/e1_rope_publication_v1.py:609-649; Q prologue :619-623; rounding contract `_rows`
// :551-582).  At head dim 256 the output accumulator alone takes 256 of the 512 TMEM columns,
// so a CTA can own only one tile:
//   TMEM   : two 64-column score buffers (columns 0..127) | O (columns 128..383) |
//            Q as 16-bit pairs (columns 384..511): the prepared Q tile is copied from shared
//            memory into TMEM once, so Q K^T takes its A operand from TMEM and only K is
//            streamed from shared memory (an SS MMA with N = 64 re-reads 4 KB of Q per
//            instruction and is shared-memory bound)
//   smem   : Q 64 KB, K ring 2 x 32 KB (64 keys x 256), V ring 2 x 32 KB; once Q is in TMEM its
//            buffer is a third ring stage (one K and one V tile) until the epilogue stages O there
//   warps  : 0-3 softmax + Q prologue + epilogue (thread r <-> row r), 4 TMA producer,
//            5 MMA issuer (one elected lane)
// At D = 128 the tile takes 256 TMEM columns (scores 128 | O 128) and 98 KB of shared memory, Q
// stays in shared memory (SS Q K^T) and two CTAs share an SM.
// The KV loop advances in sub-blocks of 64 keys with double-buffered scores exactly as in
// attn_fwd_ws.cuh: Q K^T of sub-block j+1 is queued before the issuer waits for P of sub-block
// j, P (16-bit) overwrites its score buffer and feeds O += P V from TMEM, V is an MN-major
// shared-memory operand with N = D.  CTA order: sg_decode (attn_fwd_basic.cuh) - small launches
// interleave their (batch, KV head) groups heaviest query block first, large ones only their last
// groups; the K/V tiles one CTA streams are found in L2 by its neighbours (nothing else shares
// them: no cluster multicast).
#pragma once
#include "attn_fwd_ws.cuh"

namespace kf {

constexpr int kW256Threads = 192;
constexpr int kW256KvBoxBytes = kSub * 128;           // 64 rows x 64 columns
constexpr int kW256Stages = 2;
template <int D> __host__ __device__ constexpr int ws1_q_bytes() { return (D / 64) * kBoxBytes; }            // 128 rows x D columns
template <int D> __host__ __device__ constexpr int ws1_kv_tile_bytes() { return (D / 64) * kW256KvBoxBytes; } // 64 rows x D columns
template <int D> __host__ __device__ constexpr int ws1_smem_bytes(bool factored = false) {
    // tiles, alignment slack, barriers (+ the inverse RMS of the Q rows in the factored form)
    return ws1_q_bytes<D>() + 2 * kW256Stages * ws1_kv_tile_bytes<D>() + 1024 + 512 + (factored ? 512 : 0);
}

#ifdef KF_DEBUG
// per-CTA phase stamps of thread 0 (SM clock), debug builds only
__device__ long long g_w1_time[8192 * 8];
#define KF_W1_STAMP(i) do { if (threadIdx.x == 0 && blockIdx.x < 8192) g_w1_time[blockIdx.x * 8 + (i)] = clock64(); } while (0)
#else
#define KF_W1_STAMP(i) do {} while (0)
#endif

template <int D, typename T, bool FACTORED = false>  // FACTORED: see attn_fwd_ws_kernel
__global__ void __launch_bounds__(kW256Threads, (D == 128 ? 2 : 1))
attn_fwd_ws1_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                      const AttnArgs a) {
    constexpr int NB = D / 64;                      // 64-column boxes per row
    constexpr bool kQInTmem = (D == 256);           // room for Q in TMEM only at D = 256 (one CTA per SM)
    constexpr uint32_t kTmemCols = (D == 256) ? 512 : 256;  // D = 128: two CTAs share the SM's 512 columns
    constexpr uint32_t kColO = 128;
    constexpr uint32_t kColQ = 384;  // D = 256 only: 128 columns = 256 16-bit values per row
    constexpr int kW256QBytes = ws1_q_bytes<D>();
    constexpr int kW256KvTileBytes = ws1_kv_tile_bytes<D>();
    // K/V ring: two stages of their own; at D = 256 the Q buffer, free once the prepared Q has moved to TMEM,
    // serves as a third (its 64 KB hold one K and one V tile) until the epilogue stages the output there.
    constexpr int kNS = kQInTmem ? 3 : 2;
    constexpr uint32_t kIdescQK = umma_idesc(Num<T>::kFmt, 0, kBM, kSub);
    constexpr uint32_t kIdescPV = umma_idesc(Num<T>::kFmt, 1, kBM, D);

    // An earlier CTA or launch failed: drain quickly.  One thread reads the word and the whole CTA follows that
    // reading, so no warp can leave while others go on to barriers the leaver would have served.
    KF_W1_STAMP(0);
    if (__syncthreads_or(threadIdx.x == 0 && *reinterpret_cast<volatile int*>(a.status) != 0)) return;
    KF_W1_STAMP(1);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_q = smem;
    uint8_t* smem_k = smem + kW256QBytes;
    uint8_t* smem_v = smem_k + kW256Stages * kW256KvTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem_v + kW256Stages * kW256KvTileBytes);
    // shared-memory tile of ring stage s (the third stage lives in the Q buffer)
    auto k_stage = [&](int s) { return s < kW256Stages ? smem_k + s * kW256KvTileBytes : smem_q; };
    auto v_stage = [&](int s) { return s < kW256Stages ? smem_v + s * kW256KvTileBytes : smem_q + kW256KvTileBytes; };
    uint64_t* q_full = bars + 0;
    uint64_t* q_ready = bars + 1;   // 4 arrivals (one per softmax warp)
    uint64_t* k_full = bars + 2;    // [stage]
    uint64_t* k_empty = bars + 5;   // [stage]
    uint64_t* v_full = bars + 8;    // [stage]
    uint64_t* v_empty = bars + 11;  // [stage]
    uint64_t* s_full = bars + 14;   // [buffer]
    uint64_t* p_ready = bars + 16;  // [buffer] 4 arrivals
    uint64_t* pv_done = bars + 18;  // [jj & 1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
    volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 21);
    [[maybe_unused]] float* s_inv = reinterpret_cast<float*>(bars + 64);  // [row] inverse RMS of the raw Q rows (factored form)

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- work decode
    const int G = a.Hq / a.Hkv;
    const int n_mblk = (a.S + kBM - 1) / kBM;
    const int n_sub_all = (a.S + kSub - 1) / kSub;
    const SgItem it = sg_decode(blockIdx.x, a.B * a.Hkv, a.sg_groups, a.sg_first, n_mblk, G);  // heaviest query block first
    const int b = it.grp / a.Hkv, kh = it.grp % a.Hkv;
    const int m0 = (n_mblk - 1 - it.level) * kBM;
    const int h = kh * G + it.sub;
    const int n_sub = a.causal ? min((m0 + kBM) / kSub, n_sub_all) : n_sub_all;

    if (tid == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_o);
        mbar_init(q_full, 1);
        mbar_init(q_ready, 4);
#pragma unroll
        for (int i = 0; i < kNS; ++i) {
            mbar_init(k_full + i, 1);
            mbar_init(k_empty + i, 1);
            mbar_init(v_full + i, 1);
            mbar_init(v_empty + i, 1);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mbar_init(s_full + i, 1);
            mbar_init(p_ready + i, 4);
            mbar_init(pv_done + i, 1);
        }
        *s_abort = 0;
        fence_mbar_init();
        // The raw Q tile is requested at once: its trip from DRAM then overlaps the TMEM allocation and
        // the block-wide barrier below instead of following them.
        mbar_expect_tx(q_full, kW256QBytes);
#pragma unroll
        for (int bx = 0; bx < NB; ++bx) tma_load_4d(smem_q + bx * kBoxBytes, &tm_q, q_full, bx * 64, m0, h, b);
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
    KF_W1_STAMP(2);

    int fail = 0;
    int kv_issued = 0;  // producer bookkeeping for the exit path

    if (warp < 4) {
        // =================================================== softmax, Q prologue, epilogue
        const int r = tid;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
        const int row = m0 + r;
        {
            // (all lanes of a warp wait together; the vote keeps them together if the wait runs out)
            auto wait_q = [&]() {
                const bool okq = __all_sync(0xffffffffu, mbar_wait_abortable(q_full, 0, s_abort)) != 0;
                KF_W1_STAMP(7);
                return okq;
            };
            bool ok;
            if constexpr (FACTORED) ok = q_inv_coop<D, T>(smem_q, r, a, s_inv, wait_q);
            else ok = a.fuse_q ? q_prologue_coop<D, T, 4>(smem_q, r, m0, a, wait_q) : wait_q();
            if (!ok) fail = kStatusWsQFull;
        }
        float c_row = a.scale_log2e;
        if constexpr (FACTORED) {
            // every thread of the group takes part, whatever its wait returned, and all follow the vote
            if (named_barrier_or(3, 128, fail != 0)) { if (!fail) fail = kStatusWsQFull; }
            else c_row *= s_inv[r];
        }
        const float c = c_row;
        if constexpr (kQInTmem) {
            // Every row of the tile has been transformed by some thread of this group: make that visible before
            // thread r copies row r into TMEM.  The barrier also makes the outcome of the wait uniform.
            if (named_barrier_or(2, 128, fail != 0) && !fail) fail = kStatusWsQFull;
        }
        if (!fail) {
            if constexpr (kQInTmem) {
                // thread r copies row r into TMEM columns [kColQ, kColQ + D/2)
                const uint8_t* qrow = smem_q + r * 128;
                const int sw = r & 7;
#pragma unroll
                for (int bx = 0; bx < NB; ++bx) {
                    uint32_t w[32];
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch) {
                        const uint4 u = *reinterpret_cast<const uint4*>(qrow + bx * kBoxBytes + ((ch ^ sw) << 4));
                        w[ch * 4 + 0] = u.x; w[ch * 4 + 1] = u.y; w[ch * 4 + 2] = u.z; w[ch * 4 + 3] = u.w;
                    }
                    tmem_st32(lane_base + kColQ + bx * 32, w);
                }
            } else {
                fence_proxy_async_smem();  // Q stays in shared memory as the A operand
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_ready);
        }
        float m_used = -INFINITY, den = 0.f;
        const float inv_c = 1.f / c;
        PolyBase pb;
        pb.set(0.f, inv_c);
        KF_W1_STAMP(3);
        for (int jj = 0; jj < n_sub && !fail; ++jj) {
            const int buf = jj & 1;
            const int n0 = jj * kSub;
            const uint32_t col_sb = buf * kSub;
            if (!mbar_wait_abortable(s_full + buf, (jj >> 1) & 1, s_abort)) { fail = kStatusWsSFull; break; }
            tc_fence_after();
            if (jj == 0) KF_W1_STAMP(4);
            uint32_t sr[2][32];
            tmem_ld32(lane_base + col_sb, sr[0]);
            tmem_ld32(lane_base + col_sb + 32, sr[1]);
            tmem_wait_ld();
            const bool need_mask = (n0 + kSub > a.S) || (a.causal && (n0 + kSub - 1 > m0));
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
                pb.set(m_used, inv_c);
            }
            const float neg_m = -m_used;
            const f32x2 c2 = f2_pack(c, c), nm2 = f2_pack(neg_m, neg_m);
            f32x2 psum = f2_pack(0.f, 0.f);
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
            float ps0, ps1;
            f2_unpack(psum, ps0, ps1);
            den += ps0 + ps1;
            if (jj > 0 && __any_sync(0xffffffffu, grow)) {
                // O may only be touched once the previous P V has completed.  (pv_done alternates between
                // two barriers, so a phase cannot be lapped: P V of jj+1 needs this sub-block's P.)
                if (!mbar_wait_abortable(pv_done + ((jj - 1) & 1), ((jj - 1) >> 1) & 1, s_abort)) { fail = kStatusWsPvDone; break; }
                tc_fence_after();
#pragma unroll
                for (int q4 = 0; q4 < D / 32; ++q4) {
                    uint32_t o[32];
                    tmem_ld32(lane_base + kColO + q4 * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(lane_base + kColO + q4 * 32, o);
                }
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_ready + buf);
        }
        KF_W1_STAMP(5);
        // ---- epilogue: O / den -> 16-bit -> swizzled smem (the Q buffer) -> TMA store
        if (!fail && n_sub > 0 &&
            !mbar_wait_abortable(pv_done + ((n_sub - 1) & 1), ((n_sub - 1) >> 1) & 1, s_abort)) fail = kStatusWsODone;
        if (!fail) {
            tc_fence_after();
            const float inv_den = 1.f / den;
            uint8_t* orow = smem_q + r * 128;
            const int sw = r & 7;
#pragma unroll
            for (int q4 = 0; q4 < D / 32; ++q4) {
                uint32_t o[32];
                tmem_ld32(lane_base + kColO + q4 * 32, o);
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
        named_barrier_sync(1, 128);
        if (warp == 0 && elect_one() && *s_abort == 0) {
#pragma unroll
            for (int bx = 0; bx < NB; ++bx) tma_store_4d(&tm_o, smem_q + bx * kBoxBytes, bx * 64, m0, h, b);
            tma_store_commit();
            tma_store_wait_read();  // the buffer must outlive the copy's reads; the writes drain on their own
        }
        KF_W1_STAMP(6);
    } else if (warp == 4) {
        // =================================================== TMA producer
        if (elect_one()) {
            int s = 0;
            uint32_t epar = 1;  // passes at once on the first turn of the ring
            // K is the output of the row-prepare launched just before this kernel: when this grid was launched as
            // its programmatic dependent, everything up to here (barriers, TMEM, the raw Q copy and its transform)
            // has overlapped the prepare, and the first K copy waits for it to complete.
            grid_dep_wait();
            for (int jj = 0; jj < n_sub; ++jj) {
                // (the Q buffer becomes a stage only after the prepared Q has been copied to TMEM)
                if (kNS > kW256Stages && jj == kW256Stages && !mbar_wait_abortable(q_ready, 0, s_abort)) { fail = kStatusWsQReady; break; }
                if (!mbar_wait_abortable(k_empty + s, epar, s_abort)) { fail = kStatusWsKEmpty; break; }
                mbar_expect_tx(k_full + s, kW256KvTileBytes);
                uint8_t* kd = k_stage(s);
#pragma unroll
                for (int bx = 0; bx < NB; ++bx)
                    tma_load_4d(kd + bx * kW256KvBoxBytes, &tm_k, k_full + s, bx * 64, jj * kSub, kh, b);
                if (!mbar_wait_abortable(v_empty + s, epar, s_abort)) { fail = kStatusWsVEmpty; break; }
                mbar_expect_tx(v_full + s, kW256KvTileBytes);
                uint8_t* vd = v_stage(s);
#pragma unroll
                for (int bx = 0; bx < NB; ++bx)
                    tma_load_4d(vd + bx * kW256KvBoxBytes, &tm_v, v_full + s, bx * 64, jj * kSub, kh, b);
                kv_issued = jj + 1;
                if (++s == kNS) { s = 0; epar ^= 1; }
            }
            if (fail) {
                *s_abort = 1;
                atomicCAS(a.status, 0, fail);
            }
        }
    } else {
        // =================================================== MMA issuer
        if (elect_one()) {
            const uint64_t qk_desc = umma_desc_sw128(0, 16, 1024);               // K-major operands (Q and K)
            const uint64_t v_desc = umma_desc_sw128(0, kW256KvBoxBytes, 1024);   // MN-major operand (V)
            const uint32_t qk_hi = static_cast<uint32_t>(qk_desc >> 32), v_hi = static_cast<uint32_t>(v_desc >> 32);
            uint32_t k_lo[kNS], v_lo[kNS];  // descriptor low words of the ring stages
#pragma unroll
            for (int st = 0; st < kNS; ++st) {
                k_lo[st] = static_cast<uint32_t>(qk_desc) | ((smem_u32(k_stage(st)) & 0x3FFFFu) >> 4);
                v_lo[st] = static_cast<uint32_t>(v_desc) | ((smem_u32(v_stage(st)) & 0x3FFFFu) >> 4);
            }
            const uint32_t q_lo = static_cast<uint32_t>(qk_desc) | ((smem_u32(smem_q) & 0x3FFFFu) >> 4);
            auto stage_lo = [&](const uint32_t (&lo)[kNS], int stage) {  // (no dynamic indexing of registers)
                uint32_t r = lo[0];
#pragma unroll
                for (int st = 1; st < kNS; ++st) r = (stage == st) ? lo[st] : r;
                return r;
            };
            auto issue_qk = [&](int stage, int buf) {
                const uint32_t ka = stage_lo(k_lo, stage);
                const uint32_t d = tmem_base + buf * kSub;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t kb = ka + (ks / 4) * (kW256KvBoxBytes >> 4) + (ks % 4) * 2;
                    if constexpr (kQInTmem) {
                        umma_ts_lohi(d, tmem_base + kColQ + ks * 8, kb, qk_hi, kIdescQK, ks > 0 ? 1u : 0u);
                    } else {
                        umma_ss_lohi(d, q_lo + (ks / 4) * (kBoxBytes >> 4) + (ks % 4) * 2, qk_hi, kb, qk_hi, kIdescQK,
                                     ks > 0 ? 1u : 0u);
                    }
                }
            };
            auto issue_pv = [&](int stage, int buf, uint32_t accumulate) {
                const uint32_t va = stage_lo(v_lo, stage);
                const uint32_t d = tmem_base + kColO;
                const uint32_t pa = tmem_base + buf * kSub;
                umma_ts_lohi(d, pa, va, v_hi, kIdescPV, accumulate);
#pragma unroll
                for (int ks = 1; ks < kSub / 16; ++ks) umma_ts_lohi(d, pa + ks * 8, va + ks * 128, v_hi, kIdescPV, 1u);
            };
            int kst = 0, vst = 0;
            uint32_t kpar = 0, vpar = 0;
            if (n_sub > 0 && !mbar_wait_abortable(q_ready, 0, s_abort)) fail = kStatusWsQReady;
            for (int jj = -1; jj < n_sub && !fail; ++jj) {
                const int jq = jj + 1;  // sub-block whose scores are queued now (one ahead of the P V loop)
                if (jq < n_sub) {
                    if (!mbar_wait_abortable(k_full + kst, kpar, s_abort)) { fail = kStatusWsKFull; break; }
                    tc_fence_after();
                    issue_qk(kst, jq & 1);
                    umma_commit(s_full + (jq & 1));
                    umma_commit(k_empty + kst);
                    if (++kst == kNS) { kst = 0; kpar ^= 1; }
                }
                if (jj < 0) continue;
                if (!mbar_wait_abortable(v_full + vst, vpar, s_abort)) { fail = kStatusWsVFull; break; }
                if (!mbar_wait_abortable(p_ready + (jj & 1), (jj >> 1) & 1, s_abort)) { fail = kStatusWsPReady; break; }
                tc_fence_after();
                issue_pv(vst, jj & 1, jj > 0 ? 1u : 0u);
                umma_commit(pv_done + (jj & 1));
                umma_commit(v_empty + vst);
                if (++vst == kNS) { vst = 0; vpar ^= 1; }
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
    if (warp == 4 && *s_abort != 0 && elect_one()) {
        // leave no copy in flight into this CTA's shared memory
        mbar_wait(q_full, 0);
#pragma unroll
        for (int s = 0; s < kNS; ++s) {
            if (kv_issued > s) {
                const int last_u = (kv_issued - 1 - s) / kNS;
                mbar_wait(k_full + s, last_u & 1);
                mbar_wait(v_full + s, last_u & 1);
            }
        }
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace kf
