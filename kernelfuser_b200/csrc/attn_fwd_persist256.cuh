// Persistent, warp-specialised tcgen05 flash-attention forward kernel for head dim 256.
//
// Same operator and the same inner pipeline as the D = 256 instantiation of attn_fwd_ws256.cuh (reference:
// `attention_v2_kernel`, src/e1_rope_publication_v1.py:609-649; Q prologue :619-623; rounding contract `_rows`
// :551-582): one 128-row Q tile at a time, 64-key sub-blocks, two 64-column score buffers, P over its
// scores, O (256 columns) and the prepared Q (128 columns of 16-bit pairs, the A operand of Q K^T) in TMEM.
// At this head dim a CTA owns the whole SM (512 TMEM columns, 224 KB of shared memory), so with one launch
// item per CTA nothing covers the item's fixed costs: the raw Q copy (64 KB), its RMSNorm/RoPE transform, the
// copy into TMEM, and at the end the conversion and store of a 128 x 256 output.  Here one CTA per SM takes
// tiles from a device counter, heaviest first, and a second warpgroup does that work off the main loop:
//   * the raw Q of the NEXT tile is copied into the Q buffer (free as soon as the running tile's Q is in
//     TMEM) and transformed there while the running tile computes;
//   * when the running tile's last Q K^T has completed, the next Q goes into TMEM - the tile still has a
//     sub-block of softmax and P V to go, so the next tile's first Q K^T follows its last P V directly;
//   * the finished tile's output is read from TMEM, scaled and written straight to global memory by the
//     same warpgroup (no shared-memory staging: all of it belongs to Q and the K/V ring); the next tile's
//     first P V waits only for that read.
// Roles (12 warps, registers re-balanced per warpgroup):
//   warps 0-3   softmax (thread r <-> row r <-> TMEM lane r)
//   warps 4-7   Q transform, Q -> TMEM, output epilogue
//   warp  8     K/V producer (TMA, one ring of five 64-row stages in consumption order K0 K1 V0 K2 V1 ...)
//   warp  9     MMA issuer;  warp 10  scheduler and raw-Q producer;  warp 11  spare
#pragma once
#include "attn_fwd_persist.cuh"
#include "attn_fwd_ws256.cuh"

namespace kf {

enum : int {
    kStatusP2QFree = 501, kStatusP2QFull = 502, kStatusP2QReady = 503, kStatusP2KvFull = 504, kStatusP2KvEmpty = 505,
    kStatusP2SFull = 506, kStatusP2PReady = 507, kStatusP2PvDone = 508, kStatusP2OFree = 509, kStatusP2Den = 510,
    kStatusP2Item = 511, kStatusP2QkDone = 512,
};

constexpr int kP2Threads = 384;
// Registers: the CTA starts with 168 per thread; the softmax group takes 208, the Q/epilogue group keeps 168,
// the control group gives up 40 and keeps 128.
static_assert(208 * 128 + 168 * 128 + 128 * 128 <= 168 * kP2Threads, "register re-balance must fit the launch allocation");
constexpr int kP2Ring = 5;                              // K/V ring stages
constexpr int kP2KvBoxBytes = kSub * 128;               // 64 rows x 64 columns
constexpr int kP2KvTileBytes = 4 * kP2KvBoxBytes;       // 64 rows x 256 columns (32 KB)
constexpr int kP2QBytes = 4 * kBoxBytes;                // 128 rows x 256 columns (64 KB)
#ifndef KF_P2_CLAIM_AHEAD
#define KF_P2_CLAIM_AHEAD 32
#endif
constexpr int kP2ClaimAhead = KF_P2_CLAIM_AHEAD;                        // sub-blocks before the end of a tile at which the next is claimed
constexpr int kP2SmemBytes = kP2QBytes + kP2Ring * kP2KvTileBytes + 1024 + kPsCtrlBytes;

struct P2Item {
    int b, h, kh, m0, nsub;
};

// Tile `idx` in (batch, KV head)-major order, heaviest query block first within a group.
__device__ __forceinline__ P2Item p2_decode(int idx, const AttnArgs& a) {
    P2Item it;
    const int G = a.Hq / a.Hkv;
    const int n_mblk = (a.S + kBM - 1) / kBM;
    const int n_sub_all = (a.S + kSub - 1) / kSub;
    const int upg = n_mblk * G;
    const int grp = idx / upg, r = idx % upg;
    it.b = grp / a.Hkv;
    it.kh = grp % a.Hkv;
    it.m0 = (n_mblk - 1 - r / G) * kBM;
    it.h = it.kh * G + r % G;
    it.nsub = a.causal ? min((it.m0 + kBM) / kSub, n_sub_all) : n_sub_all;
    return it;
}

struct P2Ctrl {
    uint64_t q_full;       // scheduler's TMA -> Q group: raw Q of the next tile is in the Q buffer
    uint64_t q_ready;      // Q group (4 arrivals) -> issuer: the tile's prepared Q is in TMEM
    uint64_t q_free;       // Q group (4 arrivals) -> scheduler: the Q buffer has been copied out and may be refilled
    uint64_t qk_done;      // issuer -> Q group: every Q K^T of the tile has completed (the Q columns may be overwritten)
    uint64_t kv_full[kP2Ring];
    uint64_t kv_empty[kP2Ring];
    uint64_t s_full[2];    // [buffer]
    uint64_t p_ready[2];   // [buffer] 4 arrivals
    uint64_t pv_done[2];   // [g & 1]
    uint64_t o_free;       // Q group (4 arrivals) -> issuer, softmax: the finished tile's output and row sums have been read
    uint64_t den_full;     // softmax (4 arrivals) -> Q group
    uint64_t item_full[kPsItemRing];
    uint64_t item_empty[kPsItemRing];  // 10 arrivals: 4 softmax warps, 4 Q-group warps, producer, issuer
    uint64_t near_end;     // softmax (1 arrival per tile) -> scheduler
    uint32_t tmem_slot;
    int abort_flag;
    int item[kPsItemRing];
    int dead;
    int pad[7];
    float den[kBM];
};
static_assert(sizeof(P2Ctrl) <= kPsCtrlBytes, "control block too large");

template <bool WARP>
__device__ __forceinline__ int p2_take_item(P2Ctrl* c, int n, int lane, int& fail) {
    const int s = n & (kPsItemRing - 1);
    if (!mbar_wait_abortable(c->item_full + s, (n / kPsItemRing) & 1, &c->abort_flag)) {
        fail = kStatusP2Item;
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

template <typename T>
__global__ void __launch_bounds__(kP2Threads, 1)
attn_fwd_persist256_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                           const __grid_constant__ CUtensorMap tm_v, const AttnArgs a, const int n_items) {
    constexpr int D = 256;
    constexpr int NB = D / 64;
    constexpr uint32_t kTmemCols = 512;
    constexpr uint32_t kColO = 128, kColQ = 384;
    constexpr uint32_t kIdescQK = umma_idesc(Num<T>::kFmt, 0, kBM, kSub);
    constexpr uint32_t kIdescPV = umma_idesc(Num<T>::kFmt, 1, kBM, D);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_q = smem;                       // 128 rows x 256 columns
    uint8_t* smem_kv = smem + kP2QBytes;          // [stage] 32 KB each
    P2Ctrl* c = reinterpret_cast<P2Ctrl*>(smem_kv + kP2Ring * kP2KvTileBytes);
    volatile int* s_abort = &c->abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        mbar_init(&c->q_full, 1);
        mbar_init(&c->q_ready, 4);
        mbar_init(&c->q_free, 4);
        mbar_init(&c->qk_done, 1);
        mbar_init(&c->o_free, 4);
        mbar_init(&c->den_full, 4);
        mbar_init(&c->near_end, 1);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mbar_init(c->s_full + i, 1);
            mbar_init(c->p_ready + i, 4);
            mbar_init(c->pv_done + i, 1);
        }
#pragma unroll
        for (int i = 0; i < kP2Ring; ++i) {
            mbar_init(c->kv_full + i, 1);
            mbar_init(c->kv_empty + i, 1);
        }
#pragma unroll
        for (int i = 0; i < kPsItemRing; ++i) {
            mbar_init(c->item_full + i, 1);
            mbar_init(c->item_empty + i, 10);
        }
        c->abort_flag = 0;
        // an earlier launch or CTA failed: every thread of this CTA takes the same decision from this copy
        c->dead = *reinterpret_cast<volatile int*>(a.status);
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
    const bool dead = c->dead != 0;

    int fail = 0;
    int kv_issued = 0, q_issued = 0;  // bookkeeping of the two producers for the exit path

    if (dead) {
        // nothing to do: fall through to the common exit
    } else if (warp < 4) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
        // ============================================ softmax
        const int r = tid;
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
        const float cs = a.scale_log2e;
        const float inv_c = 1.f / cs;
        int g = 0;  // sub-blocks processed so far (all tiles)
        for (int n = 0; !fail; ++n) {
            const int idx = p2_take_item<true>(c, n, lane, fail);
            if (idx < 0) break;
            const P2Item it = p2_decode(idx, a);
            const int row = it.m0 + r;
            float m_used = -INFINITY, den = 0.f;
            PolyBase pb;
            pb.set(0.f, inv_c);
            for (int jj = 0; jj < it.nsub; ++jj) {
                const int gg = g + jj;
                const int buf = gg & 1;
                const int n0 = jj * kSub;
                const uint32_t col_sb = buf * kSub;
                // tell the scheduler when this tile has only a few sub-blocks left: only then does it claim the next
                if (tid == 0 && jj == max(0, it.nsub - kP2ClaimAhead)) mbar_arrive(&c->near_end);
                if (!mbar_wait_abortable(c->s_full + buf, (gg >> 1) & 1, s_abort)) { fail = kStatusP2SFull; break; }
                tc_fence_after();
                uint32_t sr[2][32];
                tmem_ld32(lane_base + col_sb, sr[0]);
                tmem_ld32(lane_base + col_sb + 32, sr[1]);
                tmem_wait_ld();
                const bool need_mask = (n0 + kSub > a.S) || (a.causal && (n0 + kSub - 1 > it.m0));
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
                    pb.set(m_used, inv_c);
                }
                const float neg_m = -m_used;
                const f32x2 c2 = f2_pack(cs, cs), nm2 = f2_pack(neg_m, neg_m);
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
                    // O may only be touched once the previous P V has completed (pv_done alternates between two
                    // barriers, so a phase cannot be lapped: P V of g+1 needs this P)
                    if (!mbar_wait_abortable(c->pv_done + ((gg - 1) & 1), ((gg - 1) >> 1) & 1, s_abort)) { fail = kStatusP2PvDone; break; }
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
                if (lane == 0) mbar_arrive(c->p_ready + buf);
            }
            if (fail) break;
            g += it.nsub;
            // Hand the row sums to the epilogue group.  One buffer: wait until it has read the previous tile's
            // (it signals o_free after reading them); a tile of one or two sub-blocks can get here before any of
            // its P V has been issued, so this wait is not implied by the pipeline.
            if (n > 0 && !mbar_wait_abortable(&c->o_free, (n - 1) & 1, s_abort)) { fail = kStatusP2OFree; break; }
            c->den[r] = den;
            __syncwarp();
            if (lane == 0) mbar_arrive(&c->den_full);
        }
        if (fail) {
            *s_abort = 1;
            atomicCAS(a.status, 0, fail);
        }
    }
    else if (warp < 8) {
        // ============================================ Q transform, Q -> TMEM, output epilogue (keeps its 168 registers)
        const int r = tid - 128;                       // 0..127: row of the tile, TMEM lane
        const uint32_t lane_base = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
        int gsub = 0;                                  // sub-blocks of the tiles whose epilogue has been done
        // next tile: wait for its raw Q, transform it in place (RMSNorm + gamma + RoPE); returns its index or -1
        auto prepare_next = [&](int n) -> int {
            const int idx = p2_take_item<true>(c, n, lane, fail);
            if (idx < 0) return -1;
            const P2Item it = p2_decode(idx, a);
            bool waited = false, ok = true;
            auto wait_q = [&]() {
                if (waited) return ok;
                waited = true;
                // (all lanes of a warp wait here together; the vote keeps them together if the wait runs out)
                ok = __all_sync(0xffffffffu, mbar_wait_abortable(&c->q_full, n & 1, s_abort)) != 0;
                return ok;
            };
            if (a.fuse_q) q_prologue_coop<D, T, 4>(smem_q, r, it.m0, a, wait_q);
            if (!wait_q()) { fail = kStatusP2QFull; return -1; }
            return idx;
        };
        // the prepared Q moves from shared memory into TMEM columns [kColQ, kColQ + 128): thread r copies row r
        auto q_to_tmem = [&](int n) {
            // every row has been transformed by some thread of this group: make that visible to the copier
            // (the barrier also makes the outcome of the waits uniform across the group)
            if (named_barrier_or(2, 128, fail != 0)) { if (!fail) fail = kStatusP2QFull; return; }
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
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&c->q_ready);
                mbar_arrive(&c->q_free);
            }
            (void)n;
        };
        // (Waits are per thread and bounded; before the group meets at a barrier, a vote makes their outcome
        // uniform, so a wait that ran out in some threads cannot leave the others stuck at that barrier.)
        auto group_failed = [&]() {
            if (named_barrier_or(3, 128, fail != 0)) {
                if (!fail) fail = kStatusP2QFull;
                return true;
            }
            return false;
        };
        int cur = prepare_next(0);
        if (!group_failed() && cur >= 0) q_to_tmem(0);
        for (int n = 0; cur >= 0 && !fail; ++n) {
            const P2Item it = p2_decode(cur, a);
            // ---- next tile: transform its Q while this one computes, move it into TMEM once this tile's last
            // Q K^T has completed (the tile then still has a sub-block of softmax and P V to go)
            const int nxt = prepare_next(n + 1);
            if (group_failed()) break;
            if (nxt >= 0) {
                if (!mbar_wait_abortable(&c->qk_done, n & 1, s_abort)) fail = kStatusP2QkDone;
                tc_fence_after();
                q_to_tmem(n + 1);  // (its barrier makes `fail` uniform)
                if (fail) break;
            }
            // ---- epilogue of tile n: O / den -> 16-bit -> global memory
            gsub += it.nsub;
            const int gl = gsub - 1;
            {
                int f = 0;
                if (!mbar_wait_abortable(&c->den_full, n & 1, s_abort)) f = kStatusP2Den;
                else if (!mbar_wait_abortable(c->pv_done + (gl & 1), (gl >> 1) & 1, s_abort)) f = kStatusP2PvDone;
                if (f) fail = f;
                if (group_failed()) break;
            }
            tc_fence_after();
            const float inv_den = 1.f / c->den[r];
            const int row = it.m0 + r;
            T* orow = reinterpret_cast<T*>(a.out) + static_cast<long long>(it.b) * a.o_sb +
                      static_cast<long long>(it.h) * a.o_sh + static_cast<long long>(row) * a.o_ss;
            // The whole row is converted into registers first (256 16-bit values = 128 registers) so that the
            // TMEM columns are released after eight loads; the global stores follow.
            uint32_t packed[D / 2];
#pragma unroll
            for (int q4 = 0; q4 < D / 32; ++q4) {
                uint32_t o[32];
                tmem_ld32(lane_base + kColO + q4 * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    packed[q4 * 16 + i] = Num<T>::pack(__uint_as_float(o[2 * i]) * inv_den, __uint_as_float(o[2 * i + 1]) * inv_den);
            }
            // the output (and the row sums) of this tile have been read: its successor may overwrite them
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&c->o_free);
            if (row < a.S) {
#pragma unroll
                for (int ch = 0; ch < D / 8; ++ch)
                    *reinterpret_cast<uint4*>(orow + ch * 8) =
                        make_uint4(packed[ch * 4 + 0], packed[ch * 4 + 1], packed[ch * 4 + 2], packed[ch * 4 + 3]);
            }
            cur = nxt;
        }
        if (fail) {
            *s_abort = 1;
            atomicCAS(a.status, 0, fail);
        }
    }
    else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 128;");
        if (warp == 8) {
            // ============================================ K/V producer
            if (elect_one()) {
                int s = 0;            // ring stage of the next tile
                uint32_t epar = 1;    // parity to wait for on the stage's empty barrier (passes at once on the first turn)
                // next tile of the consumption order: rows [64*j, 64*j+64) of K (map tm_k) or V (map tm_v)
                auto emit = [&](const CUtensorMap* tm, int j, const P2Item& it) {
                    if (!mbar_wait_abortable(c->kv_empty + s, epar, s_abort)) { fail = kStatusP2KvEmpty; return; }
                    uint8_t* dst = smem_kv + s * kP2KvTileBytes;
                    mbar_expect_tx(c->kv_full + s, kP2KvTileBytes);
#pragma unroll
                    for (int bx = 0; bx < NB; ++bx)
                        tma_load_4d(dst + bx * kP2KvBoxBytes, tm, c->kv_full + s, bx * 64, j * kSub, it.kh, it.b);
                    ++kv_issued;
                    if (++s == kP2Ring) { s = 0; epar ^= 1; }
                };
                // (see attn_fwd_persist.cuh: the first K copy waits for the row-prepare this grid may depend on)
                grid_dep_wait();
                for (int n = 0; !fail; ++n) {
                    const int idx = p2_take_item<false>(c, n, 0, fail);
                    if (idx < 0) break;
                    const P2Item it = p2_decode(idx, a);
                    emit(&tm_k, 0, it);
                    for (int jj = 0; jj < it.nsub && !fail; ++jj) {
                        if (jj + 1 < it.nsub) emit(&tm_k, jj + 1, it);
                        if (!fail) emit(&tm_v, jj, it);
                    }
                }
                if (fail) {
                    *s_abort = 1;
                    atomicCAS(a.status, 0, fail);
                }
            }
        } else if (warp == 9) {
            // ============================================ MMA issuer
            if (elect_one()) {
                const uint32_t kv_addr = smem_u32(smem_kv);
                const uint64_t k_desc = umma_desc_sw128(0, 16, 1024);              // K-major operand (K)
                const uint64_t v_desc = umma_desc_sw128(0, kP2KvBoxBytes, 1024);   // MN-major operand (V), 8 KB between column boxes
                const uint32_t k_hi = static_cast<uint32_t>(k_desc >> 32), v_hi = static_cast<uint32_t>(v_desc >> 32);
                const uint32_t k_lo = static_cast<uint32_t>(k_desc) | ((kv_addr & 0x3FFFFu) >> 4);
                const uint32_t v_lo = static_cast<uint32_t>(v_desc) | ((kv_addr & 0x3FFFFu) >> 4);
                auto issue_qk = [&](int stage, int buf) {
                    const uint32_t ka = k_lo + stage * (kP2KvTileBytes >> 4);
                    const uint32_t d = tmem_base + buf * kSub;
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks)
                        umma_ts_lohi(d, tmem_base + kColQ + ks * 8, ka + (ks / 4) * (kP2KvBoxBytes >> 4) + (ks % 4) * 2, k_hi,
                                     kIdescQK, ks > 0 ? 1u : 0u);
                };
                auto issue_pv = [&](int stage, int buf, uint32_t accumulate) {
                    const uint32_t va = v_lo + stage * (kP2KvTileBytes >> 4);
                    const uint32_t d = tmem_base + kColO;
                    const uint32_t pa = tmem_base + buf * kSub;
                    umma_ts_lohi(d, pa, va, v_hi, kIdescPV, accumulate);
#pragma unroll
                    for (int ks = 1; ks < kSub / 16; ++ks) umma_ts_lohi(d, pa + ks * 8, va + ks * 128, v_hi, kIdescPV, 1u);
                };
                int st = 0;
                uint32_t par = 0;
                uint32_t nq = 0, np = 0;
                // scores of sub-block j of the running tile; the tile's last one also reports "every Q K^T done"
                auto take_k = [&](bool last) {
                    if (!mbar_wait_abortable(c->kv_full + st, par, s_abort)) { fail = kStatusP2KvFull; return; }
                    tc_fence_after();
                    issue_qk(st, nq & 1);
                    umma_commit(c->s_full + (nq & 1));
                    ++nq;
                    umma_commit(c->kv_empty + st);
                    if (last) umma_commit(&c->qk_done);
                    if (++st == kP2Ring) { st = 0; par ^= 1; }
                };
                for (int n = 0; !fail; ++n) {
                    const int idx = p2_take_item<false>(c, n, 0, fail);
                    if (idx < 0) break;
                    const P2Item it = p2_decode(idx, a);
                    if (!mbar_wait_abortable(&c->q_ready, n & 1, s_abort)) { fail = kStatusP2QReady; break; }
                    take_k(it.nsub == 1);
                    for (int jj = 0; jj < it.nsub && !fail; ++jj) {
                        if (jj + 1 < it.nsub) {
                            take_k(jj + 2 == it.nsub);
                            if (fail) break;
                        }
                        // ---- O += P V of sub-block jj
                        if (!mbar_wait_abortable(c->kv_full + st, par, s_abort)) { fail = kStatusP2KvFull; break; }
                        // the first P V of a tile overwrites the previous tile's output: the epilogue must have read it
                        if (jj == 0 && n > 0 && !mbar_wait_abortable(&c->o_free, (n - 1) & 1, s_abort)) { fail = kStatusP2OFree; break; }
                        if (!mbar_wait_abortable(c->p_ready + (np & 1), (np >> 1) & 1, s_abort)) { fail = kStatusP2PReady; break; }
                        tc_fence_after();
                        issue_pv(st, np & 1, jj > 0 ? 1u : 0u);
                        umma_commit(c->pv_done + (np & 1));
                        ++np;
                        umma_commit(c->kv_empty + st);
                        if (++st == kP2Ring) { st = 0; par ^= 1; }
                    }
                }
                if (fail) {
                    *s_abort = 1;
                    atomicCAS(a.status, 0, fail);
                }
            }
        } else if (warp == 10) {
            // ============================================ scheduler and raw-Q producer
            if (elect_one()) {
                for (int n = 0; !fail; ++n) {
                    // the first tile needs no counter; later ones are claimed when the running tile is about to
                    // finish (its softmax group says so), so that no CTA sits on work it cannot start yet
                    if (n > 0 && !mbar_wait_abortable(&c->near_end, (n - 1) & 1, s_abort)) { fail = kStatusP2Item; break; }
                    const int nxt = n == 0 ? static_cast<int>(blockIdx.x) : static_cast<int>(gridDim.x + atomicAdd(a.sched, 1u));
                    const int idx = nxt < n_items ? nxt : -1;
                    const int rs = n & (kPsItemRing - 1);
                    if (n >= kPsItemRing &&
                        !mbar_wait_abortable(c->item_empty + rs, (n / kPsItemRing - 1) & 1, s_abort)) { fail = kStatusP2Item; break; }
                    *reinterpret_cast<volatile int*>(c->item + rs) = idx;
                    mbar_arrive(c->item_full + rs);
                    if (idx < 0) break;
                    const P2Item it = p2_decode(idx, a);
                    // the Q buffer is free once the previous tile's prepared Q has been copied into TMEM
                    if (n > 0 && !mbar_wait_abortable(&c->q_free, (n - 1) & 1, s_abort)) { fail = kStatusP2QFree; break; }
                    mbar_expect_tx(&c->q_full, kP2QBytes);
#pragma unroll
                    for (int bx = 0; bx < NB; ++bx) tma_load_4d(smem_q + bx * kBoxBytes, &tm_q, &c->q_full, bx * 64, it.m0, it.h, it.b);
                    q_issued = n + 1;
                }
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
        if (warp == 8 && elect_one()) {
#pragma unroll
            for (int s = 0; s < kP2Ring; ++s)
                if (kv_issued > s) mbar_wait(c->kv_full + s, ((kv_issued - 1 - s) / kP2Ring) & 1);
        }
        if (warp == 10 && elect_one() && q_issued > 0) mbar_wait(&c->q_full, (q_issued - 1) & 1);
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
