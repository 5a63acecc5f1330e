// Persistent, warp-specialised tcgen05 flash-attention forward kernel (D = 128).
//
// Same operator and the same inner pipeline as attn_fwd_ws.cuh (reference:
// `attention_v2_kernel`, src/e1_rope_publication_v1.py:609-649; Q prologue
// :619-623; rounding contract `_rows` :551-582).  What changes is the life of a
// CTA: one CTA per SM takes work items (two 128-row Q tiles that share one K/V
// stream) from a device-wide counter, heaviest first, and every role keeps
// running across items.  The per-item fixed costs - the raw Q copy, its
// RMSNorm/RoPE transform, the first K/V copies, the conversion and store of the
// output - are done by other warps than the ones the main loop waits for, one
// item ahead (Q) or one item behind (output), so the tensor pipe does not idle
// between items.  The next item is claimed only when the running one has a few
// sub-blocks left: claiming earlier ties work to a CTA long before it can start
// on it, which showed as a long tail on launches of few, heavy items.
//
// Roles (16 warps, registers re-balanced per warpgroup with setmaxnreg):
//   warps 0-3 / 4-7   softmax of tile 0 / tile 1 (thread r <-> row r <-> TMEM lane r)
//   warps 8-11        Q prologue of the next item (RMSNorm + gamma + RoPE in
//                     place in shared memory) and epilogue of the finished item
//                     (O / den -> 16-bit -> swizzled smem -> TMA store)
//   warp  12          K/V producer (TMA into one ring of six 64-row stages, filled in
//                     the order the issuers consume them: K0 K1 V0 K2 V1 ...)
//   warps 13 / 14     MMA issuer of tile 0 / tile 1 (one elected lane each)
//   warp  15          scheduler (next item from the counter, published through a
//                     small ring in shared memory) and raw-Q producer (TMA)
// Shared memory: Q 2 slots x 2 tiles x 32 KB, K/V ring 6 x 16 KB (224 KB).
// TMEM (512 columns): per tile two 64-column score buffers and a 128-column
// output.  Barrier phases are derived from counters that run across items.
// Every wait is bounded and abortable as in attn_fwd_ws.cuh.
#pragma once
#include "attn_fwd_ws.cuh"

namespace kf {

enum : int {
    kStatusPsQEmpty = 301, kStatusPsQFull = 302, kStatusPsQReady = 303, kStatusPsKvFull = 304, kStatusPsKvEmpty = 305,
    kStatusPsSFull = 306, kStatusPsPReady = 307, kStatusPsPvDone = 308, kStatusPsOFree = 309, kStatusPsDen = 310,
    kStatusPsItemFull = 311, kStatusPsItemEmpty = 312,
};

// Registers per thread after the re-balance (512 threads start with 128 each; the three figures, weighted by
// 256 / 128 / 128 threads, must not exceed the 64 K registers of the SM).
#ifndef KF_PS_REG_SOFTMAX
#define KF_PS_REG_SOFTMAX 168
#define KF_PS_REG_AUX 112
#define KF_PS_REG_CTRL 64
#endif
static_assert(KF_PS_REG_SOFTMAX * 256 + KF_PS_REG_AUX * 128 + KF_PS_REG_CTRL * 128 <= 128 * 512,
              "register re-balance must fit the launch allocation (asking for more blocks forever)");
constexpr int kPsThreads = 512;
constexpr int kPsRing = 6;                        // K/V ring stages
constexpr int kPsKvTileBytes = kSub * 128 * 2;    // 64 rows x 128 columns of 16-bit values (two 8 KB boxes)
constexpr int kPsKvBoxBytes = kSub * 128;         // one 64-column x 64-row box
constexpr int kPsQSlotBytes = 2 * kWsTileBytes;   // both tiles of an item
constexpr int kPsItemRing = 4;                    // published work items in flight
// Sub-blocks before the end of an item at which the next one is claimed.  Long enough for the next item's raw
// Q copy and its transform (measured on C4 against 16: 8 is 6 % slower, 4 is 12 % slower, 32 is the same), short
// enough that no CTA sits on heavy work it cannot start (B=1 S=16384: claiming two items ahead cost 28 %).
constexpr int kPsClaimAhead = 16;
constexpr int kPsCtrlBytes = 2048;                // barriers, item ring, row sums
constexpr int kPsSmemBytes = 2 * kPsQSlotBytes + kPsRing * kPsKvTileBytes + 1024 + kPsCtrlBytes;

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

// Shared-memory control block of the persistent kernel (after the tiles).
struct PsCtrl {
    uint64_t q_full[2];      // scheduler's TMA -> prologue warps
    uint64_t q_ready[2];     // prologue warps (4 arrivals) -> issuers
    uint64_t q_empty[2];     // epilogue (1 arrival, after the output store has read the slot) -> scheduler
    uint64_t kv_full[kPsRing];
    uint64_t kv_empty[kPsRing];  // 2 arrivals (one per issuer)
    uint64_t s_full[4];      // [tile][buffer] issuer -> softmax group
    uint64_t p_ready[4];     // [tile][buffer] softmax group (4 arrivals) -> issuer
    uint64_t pv_done[4];     // [tile][g & 1] issuer -> softmax group / epilogue: P V of the tile's g-th sub-block complete
    uint64_t o_free[2];      // [tile] epilogue (4 arrivals) -> issuer: the finished item's output has left TMEM
    uint64_t den_full[2];    // [tile] softmax group (4 arrivals) -> epilogue: row sums of the finished item are in `den`
    uint64_t item_full[kPsItemRing];   // scheduler -> every role
    uint64_t item_empty[kPsItemRing];  // every role -> scheduler (15 arrivals)
    uint64_t near_end;       // softmax of tile 0 (1 arrival per item) -> scheduler: the item is about to finish
    uint32_t tmem_slot;
    int abort_flag;
    int item[kPsItemRing];
    int pad[8];
    float den[2][kBM];
};
static_assert(sizeof(PsCtrl) <= kPsCtrlBytes, "control block too large");

// Wait for the n-th published work item and return its index (< 0: no more work, or the wait failed with
// *fail set).  WARP = true: called by all lanes of a warp (one release per warp); false: by a single thread.
template <bool WARP>
__device__ __forceinline__ int ps_take_item(PsCtrl* c, int n, int lane, int& fail) {
    const int s = n & (kPsItemRing - 1);
    if (!mbar_wait_abortable(c->item_full + s, (n / kPsItemRing) & 1, &c->abort_flag)) {
        fail = kStatusPsItemFull;
        return -1;
    }
    const int idx = *reinterpret_cast<volatile int*>(c->item + s);
    if (WARP) {
        __syncwarp();
        if (lane == 0) mbar_arrive(c->item_empty + s);
    } else {
        mbar_arrive(c->item_empty + s);
    }
    return idx;
}

#ifdef KF_DEBUG
__device__ int g_ps_dbg[148 * 16 * 4];
__device__ long long g_ps_time[148 * 16 * 8];
#define KF_T0() long long dbg_t0 = clock64()
#define KF_TACC(slot) do { const long long _n = clock64(); dbg_t[slot] += _n - dbg_t0; dbg_t0 = _n; } while (0)
__device__ __forceinline__ long long dbg_gtimer() { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define KF_TDUMP() do { if (lane == 0 || warp >= 12) { dbg_t[7] = dbg_gtimer() - dbg_g0; for (int _i = 0; _i < 8; ++_i) g_ps_time[(blockIdx.x * 16 + warp) * 8 + _i] = dbg_t[_i]; } } while (0)
#define KF_DBG(nn, jj) do { dbg_n = (nn); dbg_j = (jj); } while (0)
#define KF_DBG_DUMP() do { if (lane == 0 || warp >= 12) { int* d = g_ps_dbg + (blockIdx.x * 16 + warp) * 4; d[0] = fail; d[1] = dbg_n; d[2] = dbg_j; d[3] = 1; } } while (0)
#else
#define KF_DBG(nn, jj) do {} while (0)
#define KF_DBG_DUMP() do {} while (0)
#define KF_T0() do {} while (0)
#define KF_TACC(slot) do {} while (0)
#define KF_TDUMP() do {} while (0)
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

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_q = smem;                           // [slot][tile] 32 KB each
    uint8_t* smem_kv = smem + 2 * kPsQSlotBytes;      // [stage] 16 KB each
    PsCtrl* c = reinterpret_cast<PsCtrl*>(smem_kv + kPsRing * kPsKvTileBytes);
    volatile int* s_abort = &c->abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_o);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mbar_init(c->q_full + i, 1);
            mbar_init(c->q_ready + i, 4);
            mbar_init(c->q_empty + i, 1);
            mbar_init(c->o_free + i, 4);
            mbar_init(c->den_full + i, 4);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            mbar_init(c->s_full + i, 1);
            mbar_init(c->p_ready + i, 4);
            mbar_init(c->pv_done + i, 1);
        }
#pragma unroll
        for (int i = 0; i < kPsRing; ++i) {
            mbar_init(c->kv_full + i, 1);
            mbar_init(c->kv_empty + i, 2);
        }
#pragma unroll
        for (int i = 0; i < kPsItemRing; ++i) {
            mbar_init(c->item_full + i, 1);
            mbar_init(c->item_empty + i, 15);  // 12 warps of the three warpgroup roles + K/V producer + 2 issuers
        }
        mbar_init(&c->near_end, 1);
        c->abort_flag = 0;
        // an earlier launch or CTA failed: every thread of this CTA takes the same decision from this copy
        c->pad[0] = *reinterpret_cast<volatile int*>(a.status);
        fence_mbar_init();
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(&c->tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = c->tmem_slot;
    const bool dead = c->pad[0] != 0;

    int fail = 0;
    int kv_issued = 0, q_issued = 0;  // bookkeeping of the two producers for the exit path
    [[maybe_unused]] int dbg_n = -1, dbg_j = -1;
    [[maybe_unused]] long long dbg_t[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#ifdef KF_DEBUG
    const long long dbg_g0 = dbg_gtimer();
#endif
    KF_T0();

    if (dead) {
        // nothing to do: fall through to the common exit
    } else if (warp < 8) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(KF_PS_REG_SOFTMAX));
        // ============================================ softmax of tile t
        const int t = warp >> 2;
        const int r = tid & 127;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        const uint32_t col_s = t * 128, col_o = 256 + t * 128;
        const float cs = a.scale_log2e;
        int g = 0;    // sub-blocks this tile has processed so far (all items)
        int act = 0;  // items in which this tile had work
        for (int n = 0; !fail; ++n) {
            KF_TACC(3);
            const int idx = ps_take_item<true>(c, n, lane, fail);
            if (idx < 0) break;
            KF_TACC(0);
            const PsItem it = ps_decode(idx, a);
            const int my_nsub = (t == 0) ? it.nsub[0] : it.nsub[1];
            const int my_m0 = (t == 0) ? it.m0[0] : it.m0[1];
            const int row = my_m0 + r;
            float m_used = -INFINITY, den = 0.f;
            bool s_known_ready = false;
            for (int jj = 0; jj < my_nsub; ++jj) {
                const int gg = g + jj;
                const int buf = gg & 1;
                const int n0 = jj * kSub;
                const uint32_t col_sb = col_s + buf * kSub;
                KF_DBG(n, jj);
                // tell the scheduler when this item has only a few sub-blocks left: only then does it claim the
                // next one (claiming earlier would tie work to this CTA long before it can start on it)
                if (tid == 0 && jj == max(0, my_nsub - kPsClaimAhead)) mbar_arrive(&c->near_end);
                // (usually already known from the probe issued during the previous sub-block)
                KF_TACC(2);
                if (!s_known_ready &&
                    !mbar_wait_abortable(c->s_full + 2 * t + buf, (gg >> 1) & 1, s_abort)) { fail = kStatusPsSFull; break; }
                KF_TACC(1);
                tc_fence_after();
                uint32_t sr[2][32];
                tmem_ld32(lane_base + col_sb, sr[0]);
                tmem_ld32(lane_base + col_sb + 32, sr[1]);
                tmem_wait_ld();
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
                const float m_blk = fmaxf(mx0, mx1) * cs;
                // move the exponent base only when the maximum grew by more than the threshold
                const bool grow = m_blk > m_used + kRescaleThreshold;
                float alpha = 1.f;
                if (grow) {
                    alpha = fast_exp2(m_used - m_blk);  // 0 on the first sub-block
                    m_used = m_blk;
                    den *= alpha;
                }
                const float neg_m = -m_used;
                const f32x2 c2 = f2_pack(cs, cs), nm2 = f2_pack(neg_m, neg_m);
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
                s_known_ready = (jj + 1 < my_nsub) &&
                                mbar_test_wait(c->s_full + 2 * t + (buf ^ 1), ((gg + 1) >> 1) & 1);
                float ps0, ps1;
                f2_unpack(psum, ps0, ps1);
                den += ps0 + ps1;
                if (jj > 0 && __any_sync(0xffffffffu, grow)) {
                    // O may only be touched once the previous P V has completed.  (pv_done alternates
                    // between two barriers, so a phase cannot be lapped: P V of g+1 needs this P.)
                    if (!mbar_wait_abortable(c->pv_done + 2 * t + ((gg - 1) & 1), ((gg - 1) >> 1) & 1, s_abort)) { fail = kStatusPsPvDone; break; }
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
                if (lane == 0) mbar_arrive(c->p_ready + 2 * t + buf);
            }
            if (fail) break;
            g += my_nsub;
            // Hand the row sums to the epilogue warps.  One buffer per tile: wait until the epilogue has read the
            // previous item's sums (it signals o_free after reading them).  An item of one or two sub-blocks
            // can get here before any of its P V has been issued, so this wait is not implied by the pipeline.
            // (Tiles without work in an item take no part in the hand-off: both sides count active items only.)
            if (my_nsub > 0) {
                if (act > 0 && !mbar_wait_abortable(c->o_free + t, (act - 1) & 1, s_abort)) { fail = kStatusPsOFree; break; }
                ++act;
                c->den[t][r] = den;
                __syncwarp();
                if (lane == 0) mbar_arrive(c->den_full + t);
            }
        }
        KF_DBG_DUMP();
        KF_TDUMP();
        if (fail) {
            *s_abort = 1;
            atomicCAS(a.status, 0, fail);
        }
    }
    else if (warp < 12) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(KF_PS_REG_AUX));
        // ============================================ Q prologue (two items ahead) and epilogue (one item behind)
        const int gtid = tid - 8 * 32;                 // 0..127: row of the tile, TMEM lane
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        bool more = true;                              // the scheduler has not yet published "no more work"
        int n_pro = 0;                                 // items whose prologue has been done
        int pending[2] = {-1, -1};                     // item index by slot, waiting for its epilogue
        int act[2] = {0, 0}, gsub[2] = {0, 0};         // per tile: active items and sub-blocks so far
        // prologue of the next published item: RMSNorm + gamma + RoPE of both raw Q tiles, in place
        auto prologue = [&]() {
            const int n = n_pro;
            KF_DBG(n, -100);
            const int idx = ps_take_item<true>(c, n, lane, fail);
            if (idx < 0) { more = false; return; }
            const PsItem it = ps_decode(idx, a);
            const int slot = n & 1;
            bool waited = false, ok = true;
            auto wait_q = [&]() {
                if (waited) return ok;
                waited = true;
                // (all lanes of a warp wait here together; the vote keeps them together if the wait runs out)
                ok = __all_sync(0xffffffffu, mbar_wait_abortable(c->q_full + slot, (n >> 1) & 1, s_abort));
                return ok;
            };
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                if (it.nsub[t] > 0 && a.fuse_q)
                    q_prologue_coop<D, T, 4>(smem_q + slot * kPsQSlotBytes + t * kWsTileBytes, gtid, it.m0[t], a, wait_q);
            }
            if (!wait_q()) { fail = kStatusPsQFull; return; }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(c->q_ready + slot);
            pending[slot] = idx;
            ++n_pro;
        };
        prologue();
        for (int n = 0; !fail; ++n) {
            const int slot = n & 1;
            const int idx = (slot == 0) ? pending[0] : pending[1];
            if (idx < 0) break;
            if (slot == 0) pending[0] = -1; else pending[1] = -1;
            // ---- prologue of item n + 1: it is published when item n is about to finish; its raw Q goes into
            // the other slot, which the epilogue of item n - 1 released long ago
            if (more) prologue();
            if (fail) break;
            const PsItem it = ps_decode(idx, a);
            // ---- epilogue of item n: O / den -> 16-bit -> swizzled smem (the item's Q slot) -> TMA store
#pragma unroll
            for (int t = 0; t < 2; ++t) {
                if (it.nsub[t] == 0) continue;
                gsub[t] += it.nsub[t];
                const int gl = gsub[t] - 1;  // this tile's last sub-block
                KF_DBG(n, -200 - t);
                int f = 0;
                if (!mbar_wait_abortable(c->den_full + t, act[t] & 1, s_abort)) f = kStatusPsDen;
                else if (!mbar_wait_abortable(c->pv_done + 2 * t + (gl & 1), (gl >> 1) & 1, s_abort)) f = kStatusPsPvDone;
                // (every thread of the group reaches this barrier, so a wait that ran out in some of them cannot
                // leave the others stuck at the barrier before the store)
                if (named_barrier_or(2, 128, f != 0)) { fail = f != 0 ? f : kStatusPsDen; break; }
                ++act[t];
                tc_fence_after();
                const float inv_den = 1.f / c->den[t][gtid];
                uint8_t* tile_smem = smem_q + slot * kPsQSlotBytes + t * kWsTileBytes;
                uint8_t* orow = tile_smem + gtid * 128;
                const int sw = gtid & 7;
                // The whole row is converted into registers first (128 16-bit values = 64 registers) so that the
                // TMEM columns are released after four loads; the shared-memory staging follows.
                uint32_t packed[D / 2];
#pragma unroll
                for (int q4 = 0; q4 < D / 32; ++q4) {
                    uint32_t o[32];
                    tmem_ld32(lane_base + 256 + t * 128 + q4 * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        packed[q4 * 16 + i] = Num<T>::pack(__uint_as_float(o[2 * i]) * inv_den, __uint_as_float(o[2 * i + 1]) * inv_den);
                }
                // the output (and the row sums) of this item have been read: its successor may overwrite them
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(c->o_free + t);
#pragma unroll
                for (int ch = 0; ch < D / 8; ++ch)
                    *reinterpret_cast<uint4*>(orow + (ch / 8) * kBoxBytes + (((ch % 8) ^ sw) << 4)) =
                        make_uint4(packed[ch * 4 + 0], packed[ch * 4 + 1], packed[ch * 4 + 2], packed[ch * 4 + 3]);
                fence_proxy_async_smem();
                named_barrier_sync(1, 128);
                if (gtid == 0) {
                    tma_store_4d(&tm_o, tile_smem, 0, it.m0[t], it.h[t], it.b);
                    tma_store_4d(&tm_o, tile_smem + kBoxBytes, 64, it.m0[t], it.h[t], it.b);
                    tma_store_commit();
                }
            }
            if (fail) break;
            if (gtid == 0) {
                tma_store_wait_read();  // the slot may be refilled once the copies have read it
                mbar_arrive(c->q_empty + slot);
            }
        }
        if (gtid == 0) tma_store_wait_all();
        KF_DBG_DUMP();
        if (fail) {
            *s_abort = 1;
            atomicCAS(a.status, 0, fail);
        }
    }
    else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(KF_PS_REG_CTRL));
        if (warp == 12) {
            // ============================================ K/V producer
            if (elect_one()) {
                int s = 0;            // ring stage of the next tile
                uint32_t epar = 1;    // parity to wait for on the stage's empty barrier (passes at once on the first turn)
                // next tile of the consumption order: rows [64*j, 64*j+64) of K (map tm_k) or V (map tm_v)
                auto emit = [&](const CUtensorMap* tm, int j, const PsItem& it) {
                    if (!mbar_wait_abortable(c->kv_empty + s, epar, s_abort)) { fail = kStatusPsKvEmpty; return; }
                    uint8_t* dst = smem_kv + s * kPsKvTileBytes;
                    mbar_expect_tx(c->kv_full + s, kPsKvTileBytes);
                    tma_load_4d(dst, tm, c->kv_full + s, 0, j * kSub, it.kh, it.b);
                    tma_load_4d(dst + kPsKvBoxBytes, tm, c->kv_full + s, 64, j * kSub, it.kh, it.b);
                    ++kv_issued;
                    if (++s == kPsRing) { s = 0; epar ^= 1; }
                };
                // K is the output of the row-prepare launched just before this kernel: when this grid was launched
                // as its programmatic dependent, the first K copy waits here for the prepare to complete
                grid_dep_wait();
                for (int n = 0; !fail; ++n) {
                    const int idx = ps_take_item<false>(c, n, 0, fail);
                    if (idx < 0) break;
                    const PsItem it = ps_decode(idx, a);
                    KF_DBG(n, -1);
                    if (it.n_sub > 0) emit(&tm_k, 0, it);
                    for (int jj = 0; jj < it.n_sub && !fail; ++jj) {
                        KF_DBG(n, jj);
                        if (jj + 1 < it.n_sub) emit(&tm_k, jj + 1, it);
                        if (!fail) emit(&tm_v, jj, it);
                    }
                }
                KF_DBG_DUMP();
                if (fail) {
                    *s_abort = 1;
                    atomicCAS(a.status, 0, fail);
                }
            }
        } else if (warp == 13 || warp == 14) {
            // ============================================ MMA issuer of tile t
            if (elect_one()) {
                const int t = warp - 13;
                const uint32_t q_addr = smem_u32(smem_q), kv_addr = smem_u32(smem_kv);
                // Descriptor low words in units of 16 bytes; walking a tile only adds constants:
                // +2 per 16-column K step inside a 64-column box, +1 box per 64 columns.
                const uint64_t qk_desc = umma_desc_sw128(0, 16, 1024);            // K-major operands (Q and K)
                const uint64_t v_desc = umma_desc_sw128(0, kPsKvBoxBytes, 1024);  // MN-major operand (V), 8 KB between column halves
                const uint32_t qk_hi = static_cast<uint32_t>(qk_desc >> 32), v_hi = static_cast<uint32_t>(v_desc >> 32);
                const uint32_t q_lo = static_cast<uint32_t>(qk_desc) | ((q_addr & 0x3FFFFu) >> 4);
                const uint32_t k_lo = static_cast<uint32_t>(qk_desc) | ((kv_addr & 0x3FFFFu) >> 4);
                const uint32_t v_lo = static_cast<uint32_t>(v_desc) | ((kv_addr & 0x3FFFFu) >> 4);
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
                // Running cursors instead of index arithmetic (this single thread's instruction stream is on
                // the critical path): ring stage of the next tile to consume, scores and P V issued so far.
                int st = 0;
                uint32_t par = 0;
                uint32_t nq = 0, np = 0;
                int act = 0;  // items in which this tile had work
                // (A K/V stage is waited for and released even when this tile has no work left in it, so that
                // this issuer's releases can never run a whole ring turn ahead of the other issuer's.)
                auto take_k = [&](uint32_t qa, bool mine) {
                    KF_TACC(6);
                    if (!mbar_wait_abortable(c->kv_full + st, par, s_abort)) { fail = kStatusPsKvFull; return; }
                    KF_TACC(2);
                    if (mine) {
                        tc_fence_after();
                        issue_qk(qa, st, nq & 1);
                        umma_commit(c->s_full + 2 * t + (nq & 1));
                        ++nq;
                    }
                    umma_commit(c->kv_empty + st);
                    if (++st == kPsRing) { st = 0; par ^= 1; }
                };
                for (int n = 0; !fail; ++n) {
                    KF_TACC(6);
                    const int idx = ps_take_item<false>(c, n, 0, fail);
                    if (idx < 0) break;
                    KF_TACC(0);
                    const PsItem it = ps_decode(idx, a);
                    const int my_nsub = (t == 0) ? it.nsub[0] : it.nsub[1];
                    const int n_sub = it.n_sub;
                    const int slot = n & 1;
                    const uint32_t qa = q_lo + ((slot * kPsQSlotBytes + t * kWsTileBytes) >> 4);
                    if (my_nsub > 0 && !mbar_wait_abortable(c->q_ready + slot, (n >> 1) & 1, s_abort)) { fail = kStatusPsQReady; break; }
                    KF_TACC(1);
                    KF_DBG(n, -1);
                    if (n_sub > 0) take_k(qa, my_nsub > 0);
                    for (int jj = 0; jj < n_sub && !fail; ++jj) {
                        KF_DBG(n, jj);
                        if (jj + 1 < n_sub) {
                            take_k(qa, jj + 1 < my_nsub);
                            if (fail) break;
                        }
                        // ---- O += P V of sub-block jj
                        KF_TACC(6);
                        if (!mbar_wait_abortable(c->kv_full + st, par, s_abort)) { fail = kStatusPsKvFull; break; }
                        KF_TACC(3);
                        if (jj < my_nsub) {
                            // the first P V of an item overwrites the previous item's output: the epilogue must have read it
                            if (jj == 0 && act > 0 &&
                                !mbar_wait_abortable(c->o_free + t, (act - 1) & 1, s_abort)) { fail = kStatusPsOFree; break; }
                            KF_TACC(4);
                            if (!mbar_wait_abortable(c->p_ready + 2 * t + (np & 1), (np >> 1) & 1, s_abort)) { fail = kStatusPsPReady; break; }
                            KF_TACC(5);
                            tc_fence_after();
                            issue_pv(st, np & 1, jj > 0 ? 1u : 0u);
                            umma_commit(c->pv_done + 2 * t + (np & 1));
                            ++np;
                        }
                        umma_commit(c->kv_empty + st);
                        if (++st == kPsRing) { st = 0; par ^= 1; }
                    }
                    if (my_nsub > 0) ++act;
                }
                KF_DBG_DUMP();
                KF_TDUMP();
                if (fail) {
                    *s_abort = 1;
                    atomicCAS(a.status, 0, fail);
                }
            }
        } else {
            // ============================================ scheduler and raw-Q producer
            if (elect_one()) {
                for (int n = 0; !fail; ++n) {
                    // the first item needs no counter; later ones are claimed when the running item is about to
                    // finish (its softmax group says so), so that no CTA sits on work it cannot start yet
                    if (n > 0 && !mbar_wait_abortable(&c->near_end, (n - 1) & 1, s_abort)) { fail = kStatusPsItemEmpty; break; }
                    const int nxt = n == 0 ? static_cast<int>(blockIdx.x) : static_cast<int>(gridDim.x + atomicAdd(a.sched, 1u));
                    const int idx = nxt < n_items ? nxt : -1;
                    const int rs = n & (kPsItemRing - 1);
                    KF_DBG(n, idx);
                    if (n >= kPsItemRing &&
                        !mbar_wait_abortable(c->item_empty + rs, (n / kPsItemRing - 1) & 1, s_abort)) { fail = kStatusPsItemEmpty; break; }
                    *reinterpret_cast<volatile int*>(c->item + rs) = idx;
                    mbar_arrive(c->item_full + rs);
                    if (idx < 0) break;
                    const PsItem it = ps_decode(idx, a);
                    const int slot = n & 1;
                    if (n >= 2 && !mbar_wait_abortable(c->q_empty + slot, ((n >> 1) - 1) & 1, s_abort)) { fail = kStatusPsQEmpty; break; }
                    const int active = (it.nsub[0] > 0) + (it.nsub[1] > 0);
                    mbar_expect_tx(c->q_full + slot, active * kWsTileBytes);
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        if (it.nsub[t] > 0) {
                            uint8_t* dst = smem_q + slot * kPsQSlotBytes + t * kWsTileBytes;
                            tma_load_4d(dst, &tm_q, c->q_full + slot, 0, it.m0[t], it.h[t], it.b);
                            tma_load_4d(dst + kBoxBytes, &tm_q, c->q_full + slot, 64, it.m0[t], it.h[t], it.b);
                        }
                    }
                    q_issued = n + 1;
                }
                KF_DBG_DUMP();
                if (fail) {
                    *s_abort = 1;
                    atomicCAS(a.status, 0, fail);
                }
            }
        }
    }

    // ---- common exit
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (!dead && *s_abort != 0) {
        // leave no copy in flight into this CTA's shared memory
        if (warp == 12 && elect_one()) {
#pragma unroll
            for (int s = 0; s < kPsRing; ++s)
                if (kv_issued > s) mbar_wait(c->kv_full + s, ((kv_issued - 1 - s) / kPsRing) & 1);
        }
        if (warp == 15 && elect_one()) {
#pragma unroll
            for (int s = 0; s < 2; ++s)
                if (q_issued > s) mbar_wait(c->q_full + s, ((q_issued - 1 - s) / 2) & 1);
        }
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
    // The last CTA to leave resets the work counter for the next launch that uses it.
    if (tid == 0) {
        __threadfence();
        const unsigned int left = atomicAdd(a.sched + 1, 1u);
        if (left == gridDim.x - 1) {
            a.sched[0] = 0;
            a.sched[1] = 0;
            __threadfence();
        }
    }
}

}  // namespace kf
