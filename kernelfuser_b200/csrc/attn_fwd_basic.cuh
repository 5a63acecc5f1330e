// Baseline tcgen05 flash-attention forward kernel (one 128-row Q tile per CTA).
//
// Replaces the reference's `attention_v2_kernel`
// (src/e1_rope_publication_v1.py:609-649): Q prologue (RMSNorm + gamma + RoPE,
// :619-623, rounding contract of `_rows` :551-582), KV loop with exp2 online
// softmax and causal loop bound (:624-647), epilogue O = acc / den (:648).
//
// Structure (D = 128 or 256, 16-bit type T):
//   * 128 threads; thread r owns Q row r, TMEM lane r and output row r.
//   * Q/K/V tiles arrive by TMA (4-D maps over [B,H,S,D], 64-column boxes,
//     128-byte swizzle, zero fill past the end of the sequence).
//   * The raw Q tile is normalised and rotated IN PLACE in shared memory, in
//     the swizzled layout the MMA descriptor expects (cooperatively: D/16 lanes
//     per row, coalesced table reads) - no normalised-Q tensor ever exists in
//     global memory.
//   * S = Q K^T : tcgen05.mma, A and B from shared memory (K-major),
//     accumulator in TMEM columns [0,128).
//   * P (16-bit) is written back over S in TMEM and used as the A operand of
//     O += P V, with V as an MN-major shared-memory B operand; O lives in TMEM
//     columns [128, 128+D).
//   * single K and V buffers; two CTAs per SM (D = 128) overlap each other's
//     softmax and MMA phases.
// This kernel serialises softmax and MMA inside a CTA; it is the simple,
// fully general variant (all head dims, dtypes, tails).
#pragma once
#include "ptx.cuh"
#include "rounding.cuh"

namespace kf {

struct AttnArgs {
    const void* gq;   // [D] gamma for the Q prologue
    const void* gk;   // [D] gamma for K tiles transformed inside the loop (fuse_k), else unused
    const void* cos;  // [S, D] or null
    const void* sin;  // [S, D] or null
    int B, Hq, Hkv, S;
    float scale_log2e;  // softmax scale * log2(e)
    float eps;
    int causal, rope, hf_norm, fuse_q;
    int fuse_k;    // the K operand is the RAW key tensor: every tile is normalised and rotated after it lands
    int factored;  // factored no-RoPE form: q stays raw, scores are scaled by the row's inverse RMS
    int sg_groups; // (batch, KV head) groups per super-group of the CTA order (see sg_decode)
    int sg_first;  // leading groups that run one after the other
    int* status;  // device status word: 0 = ok, else first failure code
    unsigned int* sched;  // persistent kernels: {next work item, CTAs that have left}; both 0 between launches
    void* out;            // output tensor and its element strides, for the kernel that stores rows itself
    long long o_sb, o_sh, o_ss;
};

enum : int {
    kStatusWaitQ = 101, kStatusWaitK = 102, kStatusWaitV = 103, kStatusWaitS = 104, kStatusWaitO = 105,
};

constexpr int kBM = 128;  // query rows per tile
constexpr int kBN = 128;  // keys per KV block
constexpr int kBoxBytes = 128 * 128;  // one 64-column x 128-row box of 16-bit values

template <int D> constexpr int attn_basic_smem_bytes() {
    return 3 * (D / 64) * kBoxBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Cooperative Q prologue for a group of WARPS warps (4, or 8 with gtid 0..255) on one swizzled
// 128-row tile.  D/16 lanes share a row (each owns one 16-byte chunk and its
// rotation partner), so a warp touches 32/(D/16) rows per step with coalesced
// table reads; the table chunks of the first batch of rows are fetched
// BEFORE `wait_q()` (which blocks until the raw tile has landed), so their
// latency overlaps the Q copy.  Returns false if the wait failed.
// `gamma` is the weight of the rows in the tile (Q's, or K's when a key tile is transformed in the loop) and
// `m0` the sequence position of its first row.
template <int D, typename T, int HALVES = 2, int WARPS = 4, typename WaitFn>
__device__ __forceinline__ bool rows_prologue_coop(uint8_t* smem_q, int gtid, int m0, const AttnArgs& a, const void* gamma,
                                                   WaitFn&& wait_q) {
    constexpr int LPR = D / 16;              // lanes per row
    constexpr int RPW = 32 / LPR;            // rows per warp step
    constexpr int NIT = kBM / (WARPS * RPW);     // steps
    constexpr int HALF = NIT / HALVES;       // steps whose table chunks are in flight together
    constexpr int NB = D / 64;
    const int lane = gtid & 31, w = gtid >> 5;
    const int sub = lane % LPR, rsub = lane / LPR;
    const bool hf = a.hf_norm != 0;
    const uint4* g4 = reinterpret_cast<const uint4*>(gamma);
    const uint4 glo = __ldg(g4 + sub), ghi = __ldg(g4 + LPR + sub);
    uint4 tb[HALF][4];
    auto load_tables = [&](int it0) {
#pragma unroll
        for (int i = 0; i < HALF; ++i) {
            const int pos = m0 + (it0 + i) * WARPS * RPW + w * RPW + rsub;
            if (a.rope != 0 && pos < a.S) {
                const uint4* c4 = reinterpret_cast<const uint4*>(a.cos) + static_cast<long long>(pos) * (D / 8);
                const uint4* s4 = reinterpret_cast<const uint4*>(a.sin) + static_cast<long long>(pos) * (D / 8);
                tb[i][0] = __ldg(c4 + sub);
                tb[i][1] = __ldg(c4 + LPR + sub);
                tb[i][2] = __ldg(s4 + sub);
                tb[i][3] = __ldg(s4 + LPR + sub);
            } else {
                tb[i][0] = tb[i][1] = tb[i][2] = tb[i][3] = make_uint4(0, 0, 0, 0);
            }
        }
    };
    load_tables(0);
    if (!wait_q()) return false;
#pragma unroll
    for (int h = 0; h < HALVES; ++h) {
        if (h > 0) load_tables(h * HALF);
#pragma unroll
        for (int i = 0; i < HALF; ++i) {
            const int r = (h * HALF + i) * WARPS * RPW + w * RPW + rsub;
            const bool rope = a.rope != 0 && (m0 + r) < a.S;
            uint8_t* row = smem_q + r * 128;
            const int off = ((sub % 8) ^ (r & 7)) << 4;
            uint4* plo = reinterpret_cast<uint4*>(row + (sub / 8) * kBoxBytes + off);
            uint4* phi = reinterpret_cast<uint4*>(row + (sub / 8 + NB / 2) * kBoxBytes + off);
            uint4 lo = *plo, hi = *phi;
            float ss = sumsq_chunk<T>(hi, sumsq_chunk<T>(lo, 0.f));
#pragma unroll
            for (int m = LPR / 2; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
            const float inv = rsqrtf(ss * (1.0f / static_cast<float>(D)) + a.eps);
            transform_pair<T>(lo, hi, inv, glo, ghi, tb[i][0], tb[i][1], tb[i][2], tb[i][3], hf, rope);
            *plo = lo;
            *phi = hi;
        }
    }
    return true;
}

template <int D, typename T, int HALVES = 2, int WARPS = 4, typename WaitFn>
__device__ __forceinline__ bool q_prologue_coop(uint8_t* smem_q, int gtid, int m0, const AttnArgs& a, WaitFn&& wait_q) {
    return rows_prologue_coop<D, T, HALVES, WARPS>(smem_q, gtid, m0, a, a.gq, static_cast<WaitFn&&>(wait_q));
}

// CTA order of the pipelined kernels.  The (batch, KV head) groups are cut into super-groups of
// `sg_groups` groups whose K and V together fit comfortably in L2; inside a super-group the CTAs are
// ordered heaviest query block first ACROSS its groups (all groups' last query blocks, then all
// second-to-last ones, ...), super-groups follow one another.  CTAs that run together therefore still
// stream a small set of K/V tensors through L2, while the heavy CTAs of every group start early: with
// one group after the other, the last group's heaviest CTA starts when almost no other work is left and
// becomes the tail of the launch (12 % of the time at 16 groups, 2 % at 128).  Large launches interleave only
// their last few groups (sg_first > 0): enough to keep the tail short without giving up the locality of the
// group-major order for the bulk of the launch.
//   cta            blockIdx.x
//   per_level      CTAs of one group at one query-block level (query heads, or head pairs)
//   n_levels       query-block levels per group
// Returns the group, the level counted from the heaviest (0 = last query block) and the position in it.
struct SgItem {
    int grp, level, sub;
};
__device__ __forceinline__ SgItem sg_decode(int cta, int n_groups, int sg_groups, int sg_first, int n_levels,
                                            int per_level) {
    // the first sg_first groups run one after the other (large launches interleave only their last groups)
    const int upg = n_levels * per_level;
    if (cta < sg_first * upg) {
        SgItem it;
        it.grp = cta / upg;
        const int r = cta - it.grp * upg;
        it.level = r / per_level;
        it.sub = r - it.level * per_level;
        return it;
    }
    cta -= sg_first * upg;
    n_groups -= sg_first;
    const int per_sg = sg_groups * n_levels * per_level;  // CTAs of a full super-group
    const int sg = cta / per_sg;
    const int g0 = sg * sg_groups;
    const int gs = min(sg_groups, n_groups - g0);          // groups of this super-group (the last may be short)
    const int j = cta - sg * per_sg;
    const int row = gs * per_level;                        // CTAs of one level of this super-group
    SgItem it;
    it.level = j / row;
    const int rem = j - it.level * row;
    it.grp = sg_first + g0 + rem / per_level;
    it.sub = rem % per_level;
    return it;
}

// Factored no-RoPE form (the reference's `factored_attention_kernel`,
// src/e1_qk_publication_v3.py:614-635): the query weight has been folded into the prepared keys, so
// the Q tile stays raw and only inv[r] = rsqrt(sum_j q[r,j]^2 / D + eps) is needed, which multiplies
// the row's softmax scale.  Same cooperative mapping as q_prologue_coop (D/16 lanes per row); the lane
// holding the row's first chunk stores the result.  The caller synchronises the 128 threads before
// reading inv_out.  Returns false if the wait failed.
template <int D, typename T, typename WaitFn>
__device__ __forceinline__ bool q_inv_coop(const uint8_t* smem_q, int gtid, const AttnArgs& a, float* inv_out,
                                           WaitFn&& wait_q) {
    constexpr int LPR = D / 16;
    constexpr int RPW = 32 / LPR;
    constexpr int NIT = kBM / (4 * RPW);
    constexpr int NB = D / 64;
    const int lane = gtid & 31, w = gtid >> 5;
    const int sub = lane % LPR, rsub = lane / LPR;
    if (!wait_q()) return false;
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
        const int r = it * 4 * RPW + w * RPW + rsub;
        const uint8_t* row = smem_q + r * 128;
        const int off = ((sub % 8) ^ (r & 7)) << 4;
        const uint4 lo = *reinterpret_cast<const uint4*>(row + (sub / 8) * kBoxBytes + off);
        const uint4 hi = *reinterpret_cast<const uint4*>(row + (sub / 8 + NB / 2) * kBoxBytes + off);
        float ss = sumsq_chunk<T>(hi, sumsq_chunk<T>(lo, 0.f));
#pragma unroll
        for (int m = LPR / 2; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
        if (sub == 0) inv_out[r] = rsqrtf(ss * (1.0f / static_cast<float>(D)) + a.eps);
    }
    return true;
}

template <int D, typename T>
__global__ void __launch_bounds__(128, (D == 128 ? 2 : 1))
attn_fwd_basic_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                      const AttnArgs a) {
    constexpr int NB = D / 64;
    constexpr uint32_t kTileBytes = NB * kBoxBytes;
    constexpr uint32_t kTmemCols = (D == 128) ? 256 : 512;
    constexpr uint32_t kColS = 0, kColO = 128;
    constexpr uint32_t kIdescQK = umma_idesc(Num<T>::kFmt, 0, kBM, kBN);
    constexpr uint32_t kIdescPV = umma_idesc(Num<T>::kFmt, 1, kBM, D);

    // An earlier CTA or launch failed: drain quickly.  One thread reads the word and the whole CTA follows that
    // reading, so no warp can leave while others go on to barriers the leaver would have served.
    if (__syncthreads_or(threadIdx.x == 0 && *reinterpret_cast<volatile int*>(a.status) != 0)) return;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* smem_q = smem;
    uint8_t* smem_k = smem + kTileBytes;
    uint8_t* smem_v = smem + 2 * kTileBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 3 * kTileBytes);
    uint64_t* bar_q = bars + 0;
    uint64_t* bar_k = bars + 1;
    uint64_t* bar_v = bars + 2;
    uint64_t* bar_s = bars + 3;
    uint64_t* bar_o = bars + 4;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);

    const int tid = threadIdx.x, warp = tid >> 5;

    // ---- tile decode: heavy (late) query blocks first, heads of one KV group adjacent
    const int n_mblk = (a.S + kBM - 1) / kBM;
    const int bh = a.B * a.Hq;
    const int mblk = n_mblk - 1 - static_cast<int>(blockIdx.x / bh);
    const int rem = blockIdx.x % bh;
    const int b = rem / a.Hq, h = rem % a.Hq;
    const int kh = h / (a.Hq / a.Hkv);
    const int m0 = mblk * kBM;
    const int n_kv_all = (a.S + kBN - 1) / kBN;
    const int nblk = a.causal ? min((m0 + kBM + kBN - 1) / kBN, n_kv_all) : n_kv_all;

    if (tid == 0) {
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
        prefetch_tensormap(&tm_o);
        mbar_init(bar_q, 1);
        mbar_init(bar_k, 1);
        mbar_init(bar_v, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
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
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);

    int fail = 0;
    int k_pending = 0, v_pending = 0;  // thread 0 only: a load was issued and not yet waited for
    int k_loads = 0, v_loads = 0;      // thread 0 only: loads issued so far
    if (warp == 0 && elect_one()) {
        mbar_expect_tx(bar_q, kTileBytes);
#pragma unroll
        for (int bx = 0; bx < NB; ++bx) tma_load_4d(smem_q + bx * kBoxBytes, &tm_q, bar_q, bx * 64, m0, h, b);
        mbar_expect_tx(bar_k, kTileBytes);
#pragma unroll
        for (int bx = 0; bx < NB; ++bx) tma_load_4d(smem_k + bx * kBoxBytes, &tm_k, bar_k, bx * 64, 0, kh, b);
        mbar_expect_tx(bar_v, kTileBytes);
#pragma unroll
        for (int bx = 0; bx < NB; ++bx) tma_load_4d(smem_v + bx * kBoxBytes, &tm_v, bar_v, bx * 64, 0, kh, b);
        k_pending = v_pending = 1;
        k_loads = v_loads = 1;
    }

    // ---- Q prologue
    {
        auto wait_q = [&]() { return __all_sync(0xffffffffu, mbar_wait(bar_q, 0)) != 0; };
        const bool ok = a.fuse_q ? q_prologue_coop<D, T, 4>(smem_q, tid, m0, a, wait_q) : wait_q();
        if (!ok) fail = kStatusWaitQ;
    }
    if (!fail) fence_proxy_async_smem();
    __syncthreads();

    float m_run = -INFINITY, den = 0.f;
    const int row = m0 + tid;
    const uint32_t q_addr = smem_u32(smem_q), k_addr = smem_u32(smem_k), v_addr = smem_u32(smem_v);

    for (int j = 0; j < nblk && !fail; ++j) {
        const uint32_t ph = j & 1;
        const int n0 = j * kBN;
        if (a.fuse_k) {
            // The reference's full fusion (`FUSE_K`, src/e1_rope_publication_v1.py:633-634): the tile that landed
            // is the raw K; all threads normalise and rotate it in place (positions n0 ...) before the MMA reads it.
            auto wait_k = [&]() { return __all_sync(0xffffffffu, mbar_wait(bar_k, ph)) != 0; };
            const bool ok = rows_prologue_coop<D, T, 4>(smem_k, tid, n0, a, a.gk, wait_k);
            if (ok) fence_proxy_async_smem();
            if (__syncthreads_or(!ok)) { fail = kStatusWaitK; break; }
        }
        // ---------------- S = Q K^T
        if (warp == 0 && elect_one()) {
            if (!mbar_wait(bar_k, ph)) {
                fail = kStatusWaitK;
            } else {
                k_pending = 0;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t off = (ks / 4) * kBoxBytes + (ks % 4) * 32;
                    umma_ss(tmem_base + kColS, umma_desc_sw128(q_addr + off, 16, 1024),
                            umma_desc_sw128(k_addr + off, 16, 1024), kIdescQK, ks > 0);
                }
                umma_commit(bar_s);
            }
        }
        __syncwarp();
        // (the CTA follows one outcome: a thread that left here alone would miss the barriers below)
        if (__syncthreads_or(fail != 0 || !mbar_wait(bar_s, ph))) { if (!fail) fail = kStatusWaitS; break; }
        tc_fence_after();
        if (warp == 0 && j + 1 < nblk && elect_one()) {  // K buffer is free again
            mbar_expect_tx(bar_k, kTileBytes);
#pragma unroll
            for (int bx = 0; bx < NB; ++bx)
                tma_load_4d(smem_k + bx * kBoxBytes, &tm_k, bar_k, bx * 64, n0 + kBN, kh, b);
            k_pending = 1;
            ++k_loads;
        }
        __syncwarp();

        // ---------------- online softmax on row `row`
        uint32_t sr[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(lane_base + kColS + c * 32, sr[c]);
        tmem_wait_ld();
        const bool need_mask = (n0 + kBN > a.S) || (a.causal && (n0 + kBN - 1 > m0));
        float mx = m_run;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float x = __uint_as_float(sr[c][i]) * a.scale_log2e;
                if (need_mask) {
                    const int n = n0 + c * 32 + i;
                    if (n >= a.S || (a.causal && n > row)) x = -INFINITY;
                }
                sr[c][i] = __float_as_uint(x);
                mx = fmaxf(mx, x);
            }
        }
        const float alpha = fast_exp2(m_run - mx);  // 0 on the first block (m_run = -inf)
        float psum = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t pk[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float p0 = fast_exp2(__uint_as_float(sr[c][2 * i]) - mx);
                const float p1 = fast_exp2(__uint_as_float(sr[c][2 * i + 1]) - mx);
                psum += p0 + p1;
                pk[i] = Num<T>::pack(p0, p1);
            }
            tmem_st16(lane_base + kColS + c * 16, pk);  // P overwrites S (already in registers)
        }
        den = den * alpha + psum;
        // rescale the running output unless no row of this warp moved its maximum
        if (j > 0 && !__all_sync(0xffffffffu, mx == m_run)) {
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
                uint32_t o[32];
                tmem_ld32(lane_base + kColO + c * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                tmem_st32(lane_base + kColO + c * 32, o);
            }
        }
        m_run = mx;
        tmem_wait_st();
        tc_fence_before();
        __syncthreads();

        // ---------------- O += P V
        if (warp == 0 && elect_one()) {
            tc_fence_after();
            if (!mbar_wait(bar_v, ph)) {
                fail = kStatusWaitV;
            } else {
                v_pending = 0;
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < kBN / 16; ++ks) {
                    umma_ts(tmem_base + kColO, tmem_base + kColS + ks * 8,
                            umma_desc_sw128(v_addr + ks * 2048, kBoxBytes, 1024), kIdescPV, (j > 0) || (ks > 0));
                }
                umma_commit(bar_o);
            }
        }
        __syncwarp();
        if (__syncthreads_or(fail != 0 || !mbar_wait(bar_o, ph))) { if (!fail) fail = kStatusWaitO; break; }
        tc_fence_after();
        if (warp == 0 && j + 1 < nblk && elect_one()) {  // V buffer (and S/P columns) are free again
            mbar_expect_tx(bar_v, kTileBytes);
#pragma unroll
            for (int bx = 0; bx < NB; ++bx)
                tma_load_4d(smem_v + bx * kBoxBytes, &tm_v, bar_v, bx * 64, n0 + kBN, kh, b);
            v_pending = 1;
            ++v_loads;
        }
        __syncwarp();
    }

    // ---- epilogue: O / den -> 16-bit -> swizzled smem (Q's buffer) -> TMA store
    if (!fail) {
        const float inv_den = 1.f / den;
        uint8_t* orow = smem_q + tid * 128;
        const int sw = tid & 7;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(lane_base + kColO + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(o[q4 * 8 + i]) * inv_den;
                const int col = c * 32 + q4 * 8;  // first column of this 16-byte chunk
                const int bx = col / 64, ch = (col % 64) / 8;
                *reinterpret_cast<uint4*>(orow + bx * kBoxBytes + ((ch ^ sw) << 4)) = pack8<T>(f);
            }
        }
        fence_proxy_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0 && elect_one()) {
        if (!fail) {
#pragma unroll
            for (int bx = 0; bx < NB; ++bx) tma_store_4d(&tm_o, smem_q + bx * kBoxBytes, bx * 64, m0, h, b);
            tma_store_commit();
            tma_store_wait_all();
        } else {
            // leave no copy in flight into this CTA's shared memory
            if (k_pending) mbar_wait(bar_k, (k_loads - 1) & 1);
            if (v_pending) mbar_wait(bar_v, (v_loads - 1) & 1);
        }
    }
    if (fail) atomicCAS(a.status, 0, fail);
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace kf
