// C-ABI entry points of libkf_b200 (declared in include/kf_b200.h): host-side
// argument checks, TMA tensor-map encoding and kernel launches.  No device
// allocation, no synchronisation, no exceptions across the boundary.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <utility>

#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/kf_b200.h"
#include "attn_fwd_basic.cuh"
#include "attn_fwd_ws.cuh"
#include "attn_fwd_persist.cuh"
#include "attn_fwd_persist256.cuh"
#include "attn_fwd_ws256.cuh"
#include "prepare_rows.cuh"

#ifdef KF_DEBUG
extern "C" int kf_debug_read(int* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, kf::g_ps_dbg, sizeof(int) * 148 * 16 * 4);
}
extern "C" int kf_debug_w1(long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, kf::g_w1_time, sizeof(long long) * 8192 * 8);
}
extern "C" int kf_debug_time(long long* host_out) {
    return (int)cudaMemcpyFromSymbol(host_out, kf::g_ps_time, sizeof(long long) * 148 * 16 * 8);
}
#endif

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

// `dependent`: launch as a programmatic dependent of the kernel before it in the stream (the grid may start while
// that kernel still runs and must order its reads of that kernel's output with griddepcontrol.wait).
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel_ex(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool dependent,
                             Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (dependent) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    return launch_kernel_ex(kern, grid, block, smem, st, false, std::forward<Args>(args)...);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
// Element stride of a dimension of extent n: a multiple of 8 (16 bytes), positive unless the dimension has a
// single entry.  A zero stride over n > 1 entries (an expanded / broadcast view) is refused: the TMA maps
// describe distinct rows and would walk past the allocation.
bool stride_ok(int64_t s, int64_t n) { return (s % 8) == 0 && (s > 0 || (s == 0 && n == 1)); }

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode() {
    static EncodeFn fn = nullptr;
    if (fn) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = reinterpret_cast<EncodeFn>(p);
    return fn;
}

// 4-D map over a [B, H, S, D] tensor (D contiguous); box = 64 columns x box_rows
// rows, 128-byte swizzle, out-of-range rows read as zero / are not written.
// Encoded maps are kept in a small per-thread cache keyed by everything that goes into them: a caller that
// runs the operator on the same buffers step after step (the usual case) pays for the encoding once, and the
// host time between the operator's two launches shrinks to the launches themselves.
struct MapKey {
    const void* base;
    int dtype, B, H, S, D, box_rows;
    int64_t sb, sh, ss;
    bool operator==(const MapKey& o) const {
        return base == o.base && dtype == o.dtype && B == o.B && H == o.H && S == o.S && D == o.D &&
               box_rows == o.box_rows && sb == o.sb && sh == o.sh && ss == o.ss;
    }
};
struct MapCache {
    static constexpr int kEntries = 32;
    MapKey key[kEntries];
    CUtensorMap map[kEntries];
    bool used[kEntries] = {};
    int next = 0;
};
thread_local MapCache g_maps;

int make_map(CUtensorMap* m, const void* base, int dtype, int B, int H, int S, int D, int64_t sb, int64_t sh,
             int64_t ss, int box_rows = 128) {
    const MapKey k{base, dtype, B, H, S, D, box_rows, sb, sh, ss};
    for (int i = 0; i < MapCache::kEntries; ++i)
        if (g_maps.used[i] && g_maps.key[i] == k) {
            *m = g_maps.map[i];
            return KF_OK;
        }
    EncodeFn enc = get_encode();
    if (!enc) return fail(KF_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
    // a stride of 0 (size-1 dimension) is replaced by a valid dummy
    auto st = [&](int64_t s, int64_t dflt) { return (cuuint64_t)((s > 0 ? s : dflt) * 2); };
    cuuint64_t strides[3] = {st(ss, D), st(sh, (int64_t)S * D), st(sb, (int64_t)H * S * D)};
    cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(m, dtype == KF_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                     const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(KF_ECUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    const int slot = g_maps.next;
    g_maps.next = (slot + 1) % MapCache::kEntries;
    g_maps.key[slot] = k;
    g_maps.map[slot] = *m;
    g_maps.used[slot] = true;
    return KF_OK;
}

int check_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(KF_ECUDA, "cudaGetDevice failed");
    static int cached_major[64];
    if (dev < 0 || dev >= 64) return fail(KF_ECUDA, "device ordinal %d out of range", dev);
    if (cached_major[dev] == 0) {
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess)
            return fail(KF_ECUDA, "cannot query the compute capability");
        cached_major[dev] = major;
    }
    if (cached_major[dev] != 10) return fail(KF_ENOSUP, "this library is built for sm_100a (compute capability 10.x)");
    return KF_OK;
}

int check_common(int B, int H, int S, int D, int dtype) {
    if (dtype != KF_BF16 && dtype != KF_FP16) return fail(KF_EINVAL, "dtype must be KF_BF16 or KF_FP16");
    if (D != 128 && D != 256) return fail(KF_EINVAL, "head dim must be 128 or 256 (got %d)", D);
    if (B < 1 || H < 1 || S < 1) return fail(KF_EINVAL, "B, H and S must be >= 1 (got %d, %d, %d)", B, H, S);
    return KF_OK;
}

template <int D, typename T, bool FACTORED = false> int launch_prepare(const kf::PrepareArgs& a, cudaStream_t st) {
    constexpr int RPB = (32 / (D / 16)) * (kf::kPrepThreads / 32);
    const int gx = (a.S + RPB - 1) / RPB;
    kf::PrepareArgs args = a;
    const int BH = a.B * a.H;
    int gy = (148 * 16 + gx - 1) / gx;
    if (gy < 1) gy = 1;
    if (gy > BH) gy = BH;
    int per = (BH + gy - 1) / gy;
    per = ((per + kf::kPrepUnroll - 1) / kf::kPrepUnroll) * kf::kPrepUnroll;
    gy = (BH + per - 1) / per;
    if (gy > 65535) return fail(KF_EINVAL, "too many (batch, head) pairs");
    args.bh_per_cta = per;
    kf::prepare_rows_kernel<D, T, FACTORED><<<dim3(gx, gy), kf::kPrepThreads, 0, st>>>(args);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KF_ECUDA, "prepare_rows launch failed: %s", cudaGetErrorString(e));
    return KF_OK;
}

template <int D, typename T>
int launch_attn_basic(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                      const kf::AttnArgs& a, cudaStream_t st) {
    auto kern = kf::attn_fwd_basic_kernel<D, T>;
    constexpr int smem = kf::attn_basic_smem_bytes<D>();
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(KF_ECUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    const long long n_mblk = (a.S + kf::kBM - 1) / kf::kBM;
    const long long grid = n_mblk * a.B * a.Hq;
    if (grid > 0x7fffffffLL) return fail(KF_EINVAL, "too many tiles");
    e = launch_kernel(kern, dim3((unsigned)grid), dim3(128), smem, st, mq, mk, mv, mo, a);
    if (e != cudaSuccess) return fail(KF_ECUDA, "attention launch failed: %s", cudaGetErrorString(e));
    return KF_OK;
}

template <typename T, bool FACTORED = false>
int launch_attn_ws(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                   const kf::AttnArgs& a, cudaStream_t st) {
    auto kern = kf::attn_fwd_ws_kernel<T, FACTORED>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (FACTORED ? kf::kWsSmemBytesFactored : kf::kWsSmemBytes));
    if (e != cudaSuccess) return fail(KF_ECUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    const int G = a.Hq / a.Hkv;
    const long long n_mblk = (a.S + kf::kBM - 1) / kf::kBM;
    const long long upg = (G % 2 == 0) ? n_mblk * (G / 2) : ((n_mblk + 1) / 2) * G;
    const long long grid = upg * a.B * a.Hkv;
    if (grid > 0x7fffffffLL) return fail(KF_EINVAL, "too many tiles");
    e = launch_kernel(kern, dim3((unsigned)grid), dim3(kf::kWsThreads),
                      (size_t)(FACTORED ? kf::kWsSmemBytesFactored : kf::kWsSmemBytes), st, mq, mk, mv, mo, a);
    if (e != cudaSuccess) return fail(KF_ECUDA, "attention launch failed: %s", cudaGetErrorString(e));
    return KF_OK;
}

template <int D, typename T, bool FACTORED = false>
int launch_attn_ws1(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                    const kf::AttnArgs& a, cudaStream_t st, bool dependent = false) {
    auto kern = kf::attn_fwd_ws1_kernel<D, T, FACTORED>;
    constexpr int smem = kf::ws1_smem_bytes<D>(FACTORED);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(KF_ECUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    const long long n_mblk = (a.S + kf::kBM - 1) / kf::kBM;
    const long long grid = n_mblk * a.B * a.Hq;
    if (grid > 0x7fffffffLL) return fail(KF_EINVAL, "too many tiles");
    e = launch_kernel_ex(kern, dim3((unsigned)grid), dim3(kf::kW256Threads), (size_t)smem, st, dependent, mq, mk, mv, mo, a);
    if (e != cudaSuccess) return fail(KF_ECUDA, "attention launch failed: %s", cudaGetErrorString(e));
    return KF_OK;
}

// K + V bytes of the groups whose CTAs are interleaved heaviest-first (a fraction of the 126 MB L2).
constexpr long long kSuperGroupBytes = 48LL << 20;
// Launches of up to this many CTAs per resident slot interleave their groups.
constexpr long long kInterleaveMaxCtasPerSlot = 10;

// The one-tile kernel starts as a programmatic dependent of the row-prepare made by the same call: the prepare's
// tail and the launch gap then hide behind the attention kernel's own start-up (barriers, TMEM, raw Q copy, Q
// transform); only its first K copy waits for the prepare (griddepcontrol.wait).  Measured under graph replay:
// -17 % at B=1 S=128, -10 % at B=1 S=512, -3 % on C2 (B=1 S=2048), -0.7 % on the 8- and 4-GPU shards of C4;
// identical results.  The limit (in 128-row query tiles) exists for experiments; every launch qualifies.
#ifndef KF_DEPENDENT_MAX_TILES
#define KF_DEPENDENT_MAX_TILES (1LL << 40)
#endif
constexpr long long kDependentMaxTiles = KF_DEPENDENT_MAX_TILES;
#ifndef KF_DEPENDENT_PERSIST
#define KF_DEPENDENT_PERSIST 1
#endif

// Sub-blocks of work per SM from which variant 0 picks the persistent kernel at D = 256.
constexpr long long kPersist256MinSubBlocksPerSm = 200;

// Variant 0 at D = 128 picks the persistent two-tile kernel from this many 128-row query tiles, for sequence
// lengths strictly between the two limits below, and the one-tile-per-CTA kernel everywhere else.
constexpr long long kAutoPersistMinTiles = 8192;
constexpr int kAutoPersistMinS = 2048, kAutoPersistMaxS = 8192;

int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// Work counters of the persistent kernel: {next item, CTAs that have left} per slot.  They live in the
// library image (zero at load), the kernel's last CTA puts them back to zero, and launches take the slots in
// turn, so that launches in flight on different streams of a device do not share one (up to kSchedSlots of them).
constexpr int kSchedSlots = 64;
__device__ unsigned int g_sched[kSchedSlots][2];

int sched_slot(unsigned int** out) {
    static std::atomic<unsigned int*> base[64];
    static std::atomic<unsigned int> turn{0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(KF_ECUDA, "cudaGetDevice failed");
    unsigned int* bp = base[dev].load(std::memory_order_acquire);
    if (bp == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_sched);
        if (e != cudaSuccess || p == nullptr)
            return fail(KF_ECUDA, "cudaGetSymbolAddress(work counters) failed: %s", cudaGetErrorString(e));
        bp = static_cast<unsigned int*>(p);
        base[dev].store(bp, std::memory_order_release);
    }
    *out = bp + 2 * (turn.fetch_add(1, std::memory_order_relaxed) % kSchedSlots);
    return KF_OK;
}

template <typename T>
int launch_attn_persist(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mo,
                        const kf::AttnArgs& a0, cudaStream_t st, bool dependent = false) {
    auto kern = kf::attn_fwd_persist_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kf::kPsSmemBytes);
    if (e != cudaSuccess) return fail(KF_ECUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    kf::AttnArgs a = a0;
    if (int r = sched_slot(&a.sched)) return r;
    const int G = a.Hq / a.Hkv;
    const long long n_mblk = (a.S + kf::kBM - 1) / kf::kBM;
    const long long upg = (G % 2 == 0) ? n_mblk * (G / 2) : ((n_mblk + 1) / 2) * G;
    const long long items = upg * a.B * a.Hkv;
    if (items > 0x7fffffffLL) return fail(KF_EINVAL, "too many tiles");
    const int grid = (int)(items < sm_count() ? items : sm_count());
    e = launch_kernel_ex(kern, dim3((unsigned)grid), dim3(kf::kPsThreads), (size_t)kf::kPsSmemBytes, st, dependent, mq, mk, mv,
                         mo, a, (int)items);
    if (e != cudaSuccess) return fail(KF_ECUDA, "attention launch failed: %s", cudaGetErrorString(e));
    return KF_OK;
}

template <typename T>
int launch_attn_persist256(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const kf::AttnArgs& a0,
                           cudaStream_t st, bool dependent = false) {
    auto kern = kf::attn_fwd_persist256_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kf::kP2SmemBytes);
    if (e != cudaSuccess) return fail(KF_ECUDA, "cudaFuncSetAttribute failed: %s", cudaGetErrorString(e));
    kf::AttnArgs a = a0;
    if (int r = sched_slot(&a.sched)) return r;
    const long long n_mblk = (a.S + kf::kBM - 1) / kf::kBM;
    const long long items = n_mblk * a.B * a.Hq;
    if (items > 0x7fffffffLL) return fail(KF_EINVAL, "too many tiles");
    const int grid = (int)(items < sm_count() ? items : sm_count());
    e = launch_kernel_ex(kern, dim3((unsigned)grid), dim3(kf::kP2Threads), (size_t)kf::kP2SmemBytes, st, dependent, mq, mk, mv, a,
                         (int)items);
    if (e != cudaSuccess) return fail(KF_ECUDA, "attention launch failed: %s", cudaGetErrorString(e));
    return KF_OK;
}

}  // namespace


namespace {

int prepare_impl(const void* x, void* y, const void* gamma, const void* gamma2, const void* cos_table,
                 const void* sin_table, int B,
                    int H, int S, int D, int dtype, int hf_norm, float eps, int64_t x_sb, int64_t x_sh, int64_t x_ss,
                    int64_t y_sb, int64_t y_sh, int64_t y_ss, void* stream) {
    if (int r = check_common(B, H, S, D, dtype)) return r;
    if (!x || !y || !gamma) return fail(KF_EINVAL, "x, y and gamma must not be NULL");
    if (gamma2 && (cos_table || sin_table)) return fail(KF_EINVAL, "the factored form has no rotary tables");
    if (!aligned16(gamma2)) return fail(KF_EALIGN, "pointers must be 16-byte aligned");
    if ((cos_table == nullptr) != (sin_table == nullptr))
        return fail(KF_EINVAL, "provide both rotary tables or neither");
    if (!aligned16(x) || !aligned16(y) || !aligned16(gamma) || !aligned16(cos_table) || !aligned16(sin_table))
        return fail(KF_EALIGN, "pointers must be 16-byte aligned");
    if (!stride_ok(x_sb, B) || !stride_ok(x_sh, H) || !stride_ok(x_ss, S) || !stride_ok(y_sb, B) ||
        !stride_ok(y_sh, H) || !stride_ok(y_ss, S))
        return fail(KF_EALIGN, "strides must be positive multiples of 8 elements (0 only for a dimension of size 1)");
    if (x_ss < D || y_ss < D) return fail(KF_EINVAL, "row stride must be at least D");
    if (int r = check_device()) return r;
    kf::PrepareArgs a{};
    a.x = x; a.y = y; a.gamma = gamma; a.gamma2 = gamma2; a.cos = cos_table; a.sin = sin_table;
    a.x_sb = x_sb; a.x_sh = x_sh; a.x_ss = x_ss; a.y_sb = y_sb; a.y_sh = y_sh; a.y_ss = y_ss;
    a.B = B; a.H = H; a.S = S; a.eps = eps; a.rope = cos_table != nullptr; a.hf_norm = hf_norm != 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (gamma2) {
        if (D == 128)
            return dtype == KF_BF16 ? launch_prepare<128, __nv_bfloat16, true>(a, st)
                                    : launch_prepare<128, __half, true>(a, st);
        return dtype == KF_BF16 ? launch_prepare<256, __nv_bfloat16, true>(a, st) : launch_prepare<256, __half, true>(a, st);
    }
    if (D == 128) return dtype == KF_BF16 ? launch_prepare<128, __nv_bfloat16>(a, st) : launch_prepare<128, __half>(a, st);
    return dtype == KF_BF16 ? launch_prepare<256, __nv_bfloat16>(a, st) : launch_prepare<256, __half>(a, st);
}

int attention_impl(const void* q, const void* kn, const void* v, const void* gamma_q, const void* cos_table,
                     const void* sin_table, void* out, int B, int Hq, int Hkv, int S, int D, int dtype, int causal,
                     int hf_norm, int fuse_q, float eps, float scale, int64_t q_sb, int64_t q_sh, int64_t q_ss,
                     int64_t k_sb, int64_t k_sh, int64_t k_ss, int64_t v_sb, int64_t v_sh, int64_t v_ss,
                     int64_t o_sb, int64_t o_sh, int64_t o_ss, int* status, int variant, int factored, void* stream,
                     const void* gamma_k_full = nullptr, bool after_prepare = false) {
    // after_prepare: the launch before this one in the stream is the row-prepare that wrote `kn`, made by the same
    // call; small launches of the one-tile kernel then start as its programmatic dependent.
    // gamma_k_full != NULL: `kn` is the RAW key tensor and every K tile is normalised and rotated inside the loop
    // (the reference's mode 'full'); that form exists in the baseline kernel only.
    if (int r = check_common(B, Hq, S, D, dtype)) return r;
    if (Hkv < 1 || Hq % Hkv != 0) return fail(KF_EINVAL, "Hq (%d) must be a positive multiple of Hkv (%d)", Hq, Hkv);
    if (!q || !kn || !v || !out || !status) return fail(KF_EINVAL, "q, kn, v, out and status must not be NULL");
    if (fuse_q && !gamma_q) return fail(KF_EINVAL, "gamma_q is required when fuse_q is set");
    if ((cos_table == nullptr) != (sin_table == nullptr))
        return fail(KF_EINVAL, "provide both rotary tables or neither");
    if (!aligned16(q) || !aligned16(kn) || !aligned16(v) || !aligned16(out) || !aligned16(gamma_q) ||
        !aligned16(cos_table) || !aligned16(sin_table))
        return fail(KF_EALIGN, "pointers must be 16-byte aligned");
    const int64_t strides[12] = {q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_sb, o_sh, o_ss};
    const int64_t extents[12] = {B, Hq, S, B, Hkv, S, B, Hkv, S, B, Hq, S};
    for (int i = 0; i < 12; ++i)
        if (!stride_ok(strides[i], extents[i]))
            return fail(KF_EALIGN, "strides must be positive multiples of 8 elements (0 only for a dimension of size 1)");
    if (q_ss < D || k_ss < D || v_ss < D || o_ss < D) return fail(KF_EINVAL, "row stride must be at least D");
    if (!(scale > 0.f) || !(scale < 1e30f)) return fail(KF_EINVAL, "scale must be positive and finite");
    if (variant < 0 || variant > 5 || variant == 4) return fail(KF_EINVAL, "variant must be 0, 1, 2, 3 or 5");
    if (gamma_k_full) {
        if (!aligned16(gamma_k_full)) return fail(KF_EALIGN, "pointers must be 16-byte aligned");
        if (!fuse_q || factored) return fail(KF_EINVAL, "full fusion transforms both Q and K in the kernel");
        variant = 1;
    }
    if (int r = check_device()) return r;

    CUtensorMap mq, mk, mv, mo;
    if (int r = make_map(&mq, q, dtype, B, Hq, S, D, q_sb, q_sh, q_ss)) return r;
    if (int r = make_map(&mk, kn, dtype, B, Hkv, S, D, k_sb, k_sh, k_ss)) return r;
    if (int r = make_map(&mv, v, dtype, B, Hkv, S, D, v_sb, v_sh, v_ss)) return r;
    if (int r = make_map(&mo, out, dtype, B, Hq, S, D, o_sb, o_sh, o_ss)) return r;

    kf::AttnArgs a{};
    a.gq = gamma_q; a.cos = cos_table; a.sin = sin_table;
    a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.S = S;
    a.scale_log2e = scale * 1.4426950408889634f;
    a.eps = eps; a.causal = causal != 0; a.rope = cos_table != nullptr; a.hf_norm = hf_norm != 0;
    a.fuse_q = fuse_q != 0; a.status = status;
    a.gk = gamma_k_full; a.fuse_k = gamma_k_full != nullptr;
    a.factored = factored != 0;
    a.out = out; a.o_sb = o_sb; a.o_sh = o_sh; a.o_ss = o_ss;
    if (factored && (cos_table || sin_table)) return fail(KF_EINVAL, "the factored form has no rotary tables");
    if (factored && variant != 0 && variant != 2 && variant != 5)
        return fail(KF_EINVAL, "the factored form runs on kernels 0, 2 and 5 only");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool dependent = after_prepare && (long long)B * Hq * ((S + kf::kBM - 1) / kf::kBM) <= kDependentMaxTiles;
    // Automatic choice at D = 128.  The one-tile-per-CTA kernel (two CTAs per SM, groups interleaved heaviest
    // first) fills the SMs, keeps the causal tail short and has the better steady state (two independent CTAs
    // instead of two tiles in step): measured on B200 it is 3-9 % faster than the persistent two-tile kernel at
    // S <= 2048 and S >= 8192 whatever the size of the launch, and 1-17 % faster on launches below about eight
    // thousand query tiles.  In between (S = 3072 ... 6144 with at least 8192 tiles, C4 and its 2-GPU shard among
    // them) the persistent kernel wins by 2-6 %: it hides the per-tile fixed costs, which weigh most there, and
    // its tile pair shares one K/V stream.  (The factored form exists for kernels 2 and 5 only.)
    if (D == 128 && variant == 0) {
        const long long tiles = (long long)B * Hq * ((S + kf::kBM - 1) / kf::kBM);
        const bool mid = S > kAutoPersistMinS && S < kAutoPersistMaxS;
        if (factored) variant = tiles > kAutoPersistMinTiles ? 2 : 5;
        else variant = (tiles >= kAutoPersistMinTiles && mid) ? 3 : 5;
    }
    if (D == 128 && variant == 3) {
        CUtensorMap mk64, mv64;  // the persistent kernel streams K/V in 64-row tiles
        if (int r = make_map(&mk64, kn, dtype, B, Hkv, S, D, k_sb, k_sh, k_ss, 64)) return r;
        if (int r = make_map(&mv64, v, dtype, B, Hkv, S, D, v_sb, v_sh, v_ss, 64)) return r;
        return dtype == KF_BF16 ? launch_attn_persist<__nv_bfloat16>(mq, mk64, mv64, mo, a, st, dependent && KF_DEPENDENT_PERSIST)
                                : launch_attn_persist<__half>(mq, mk64, mv64, mo, a, st, dependent && KF_DEPENDENT_PERSIST);
    }
    {
        // CTA order (sg_decode).  Small launches - up to about ten CTAs per resident slot - interleave all
        // their (batch, KV head) groups heaviest query block first, as far as the groups' K and V stay within
        // kSuperGroupBytes of L2: otherwise the last group's heaviest CTA starts when almost nothing else is
        // left and sticks out at the end (measured: 5-17 % of such a launch).  Large launches keep one group
        // after the other: there the tail is small and interleaving costs 1-3 % of L2 locality.
        const long long groups = (long long)B * Hkv;
        const long long n_mblk = (S + kf::kBM - 1) / kf::kBM;
        const int G = Hq / Hkv;
        long long ctas_per_group = n_mblk * G;  // one 128-row tile per CTA
        long long slots = sm_count();           // CTAs resident at a time
        if (D == 128 && variant == 5) slots *= 2;
        // (the two-tiles-per-CTA kernel of D = 128 only serves large launches and keeps the group-major order)
        long long fit = kSuperGroupBytes / (2LL * S * D * 2);  // K and V of one group, bytes
        if (fit < 1) fit = 1;
        a.sg_groups = 1;
        a.sg_first = 0;
        if (causal && groups * ctas_per_group <= kInterleaveMaxCtasPerSlot * slots) {
            const long long n_sg = (groups + fit - 1) / fit;
            a.sg_groups = (int)((groups + n_sg - 1) / n_sg);
        } else if (causal) {
            // Only the last groups are interleaved: as many as give every slot about the work of the heaviest
            // CTA (twice the average CTA of a causal group).
            long long tail = (2 * slots + ctas_per_group - 1) / ctas_per_group;
            if (tail > fit) tail = fit;
            if (tail > groups) tail = groups;
            if (tail > 1) {
                a.sg_groups = (int)tail;
                a.sg_first = (int)(groups - tail);
            }
        }
    }
    if (D == 128 && variant == 5) {
        CUtensorMap mk64, mv64;  // K/V stream in 64-row tiles
        if (int r = make_map(&mk64, kn, dtype, B, Hkv, S, D, k_sb, k_sh, k_ss, 64)) return r;
        if (int r = make_map(&mv64, v, dtype, B, Hkv, S, D, v_sb, v_sh, v_ss, 64)) return r;
        if (factored)
            return dtype == KF_BF16 ? launch_attn_ws1<128, __nv_bfloat16, true>(mq, mk64, mv64, mo, a, st, dependent)
                                    : launch_attn_ws1<128, __half, true>(mq, mk64, mv64, mo, a, st, dependent);
        return dtype == KF_BF16 ? launch_attn_ws1<128, __nv_bfloat16>(mq, mk64, mv64, mo, a, st, dependent)
                                : launch_attn_ws1<128, __half>(mq, mk64, mv64, mo, a, st, dependent);
    }
    if (D == 128 && variant == 2) {
        if (factored)
            return dtype == KF_BF16 ? launch_attn_ws<__nv_bfloat16, true>(mq, mk, mv, mo, a, st)
                                    : launch_attn_ws<__half, true>(mq, mk, mv, mo, a, st);
        return dtype == KF_BF16 ? launch_attn_ws<__nv_bfloat16>(mq, mk, mv, mo, a, st)
                                : launch_attn_ws<__half>(mq, mk, mv, mo, a, st);
    }
    if (D == 256 && variant == 0 && !factored) {
        // The persistent kernel hides a tile's fixed costs (raw Q copy, transform, copy into TMEM, output store)
        // behind the previous / next tile's main loop; it pays once every SM has a few hundred 64-key sub-blocks
        // to work through (measured: -11 % time on C5, -2 ... -6 % on its 8/4-GPU shards, +4 ... +18 % on launches
        // with about a hundred sub-blocks per SM, where the one-launch-per-tile kernel balances better).
        const long long n_mblk = (S + kf::kBM - 1) / kf::kBM, n_sub_all = (S + kf::kSub - 1) / kf::kSub;
        const long long per_head = causal ? n_mblk * (n_mblk + 1) : n_mblk * n_sub_all;
        if ((long long)B * Hq * per_head >= kPersist256MinSubBlocksPerSm * sm_count()) variant = 3;
    }
    if (D == 256 && variant == 3) {
        if (factored) return fail(KF_EINVAL, "the factored form runs on kernels 0, 2 and 5 only");
        CUtensorMap mk64, mv64;  // K/V stream in 64-row tiles
        if (int r = make_map(&mk64, kn, dtype, B, Hkv, S, D, k_sb, k_sh, k_ss, 64)) return r;
        if (int r = make_map(&mv64, v, dtype, B, Hkv, S, D, v_sb, v_sh, v_ss, 64)) return r;
        return dtype == KF_BF16 ? launch_attn_persist256<__nv_bfloat16>(mq, mk64, mv64, a, st, dependent && KF_DEPENDENT_PERSIST)
                                : launch_attn_persist256<__half>(mq, mk64, mv64, a, st, dependent && KF_DEPENDENT_PERSIST);
    }
    if (D == 256 && (variant == 0 || variant == 2)) {
        CUtensorMap mk64, mv64;  // K/V stream in 64-row tiles
        if (int r = make_map(&mk64, kn, dtype, B, Hkv, S, D, k_sb, k_sh, k_ss, 64)) return r;
        if (int r = make_map(&mv64, v, dtype, B, Hkv, S, D, v_sb, v_sh, v_ss, 64)) return r;
        if (factored)
            return dtype == KF_BF16 ? launch_attn_ws1<256, __nv_bfloat16, true>(mq, mk64, mv64, mo, a, st, dependent)
                                    : launch_attn_ws1<256, __half, true>(mq, mk64, mv64, mo, a, st, dependent);
        return dtype == KF_BF16 ? launch_attn_ws1<256, __nv_bfloat16>(mq, mk64, mv64, mo, a, st, dependent)
                                : launch_attn_ws1<256, __half>(mq, mk64, mv64, mo, a, st, dependent);
    }
    if (variant >= 2) return fail(KF_EINVAL, "variant 5 supports head dim 128 only");  // D == 256 here
    if (D == 128)
        return dtype == KF_BF16 ? launch_attn_basic<128, __nv_bfloat16>(mq, mk, mv, mo, a, st)
                                : launch_attn_basic<128, __half>(mq, mk, mv, mo, a, st);
    return dtype == KF_BF16 ? launch_attn_basic<256, __nv_bfloat16>(mq, mk, mv, mo, a, st)
                            : launch_attn_basic<256, __half>(mq, mk, mv, mo, a, st);
}

}  // namespace

namespace kf {
constexpr int kStatusSelfTestWait = 901;
// One warp waits on a barrier that nobody will ever arrive on, with the same polling loop as the kernels'
// waits but a caller-given limit; when the limit runs out it records its code in the status word and
// returns.  Nothing faults, traps or hangs: this is the failure path of every bounded wait in this library,
// taken on purpose.
__global__ void selftest_wait_kernel(int* status, long long limit_clocks) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    bool ok = mbar_try_wait(&bar, 0);
    const long long t0 = clock64();
    while (!ok && clock64() - t0 <= limit_clocks) ok = mbar_try_wait(&bar, 0);
    ok = __all_sync(0xffffffffu, ok) != 0;
    if (!ok && threadIdx.x == 0) atomicCAS(status, 0, kStatusSelfTestWait);
}
}  // namespace kf

extern "C" {

int kf_version(void) { return 102; }

int kf_selftest_wait_timeout(int* status, long long limit_clocks, void* stream) {
    if (!status) return fail(KF_EINVAL, "status must not be NULL");
    if (limit_clocks < 1 || limit_clocks > (1ll << 31)) return fail(KF_EINVAL, "limit_clocks must be in [1, 2^31]");
    if (int r = check_device()) return r;
    kf::selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status, limit_clocks);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(KF_ECUDA, "self-test launch failed: %s", cudaGetErrorString(e));
    return KF_OK;
}

const char* kf_last_error(void) { return g_err; }

int kf_prepare_rows(const void* x, void* y, const void* gamma, const void* cos_table, const void* sin_table, int B,
                    int H, int S, int D, int dtype, int hf_norm, float eps, int64_t x_sb, int64_t x_sh, int64_t x_ss,
                    int64_t y_sb, int64_t y_sh, int64_t y_ss, void* stream) {
    return prepare_impl(x, y, gamma, nullptr, cos_table, sin_table, B, H, S, D, dtype, hf_norm, eps, x_sb, x_sh, x_ss,
                        y_sb, y_sh, y_ss, stream);
}

int kf_attention_fwd(const void* q, const void* kn, const void* v, const void* gamma_q, const void* cos_table,
                     const void* sin_table, void* out, int B, int Hq, int Hkv, int S, int D, int dtype, int causal,
                     int hf_norm, int fuse_q, float eps, float scale, int64_t q_sb, int64_t q_sh, int64_t q_ss,
                     int64_t k_sb, int64_t k_sh, int64_t k_ss, int64_t v_sb, int64_t v_sh, int64_t v_ss,
                     int64_t o_sb, int64_t o_sh, int64_t o_ss, int* status, int variant, void* stream) {
    return attention_impl(q, kn, v, gamma_q, cos_table, sin_table, out, B, Hq, Hkv, S, D, dtype, causal, hf_norm,
                          fuse_q, eps, scale, q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_sb, o_sh, o_ss,
                          status, variant, /*factored=*/0, stream);
}

// The whole operator in one call: row-prepare of K into the caller's `kn`, then the attention kernel - the
// reference's `launch_attention(mode='query')` (src/e1_rope_publication_v1.py:661-677).  Where the one-tile
// kernel serves the launch it starts as a programmatic dependent of the prepare (see kDependentMaxTiles).
int kf_optimized_attention(const void* q, const void* k, const void* v, const void* gamma_q, const void* gamma_k,
                           const void* cos_table, const void* sin_table, void* kn, void* out, int B, int Hq, int Hkv,
                           int S, int D, int dtype, int causal, int hf_norm, float eps, float scale, int64_t q_sb,
                           int64_t q_sh, int64_t q_ss, int64_t k_sb, int64_t k_sh, int64_t k_ss, int64_t v_sb,
                           int64_t v_sh, int64_t v_ss, int64_t n_sb, int64_t n_sh, int64_t n_ss, int64_t o_sb,
                           int64_t o_sh, int64_t o_ss, int* status, int variant, void* stream) {
    if (!gamma_q || !gamma_k) return fail(KF_EINVAL, "gamma_q and gamma_k must not be NULL");
    if (int r = prepare_impl(k, kn, gamma_k, nullptr, cos_table, sin_table, B, Hkv, S, D, dtype, hf_norm, eps, k_sb,
                             k_sh, k_ss, n_sb, n_sh, n_ss, stream))
        return r;
    return attention_impl(q, kn, v, gamma_q, cos_table, sin_table, out, B, Hq, Hkv, S, D, dtype, causal, hf_norm,
                                 /*fuse_q=*/1, eps, scale, q_sb, q_sh, q_ss, n_sb, n_sh, n_ss, v_sb, v_sh, v_ss, o_sb,
                                 o_sh, o_ss, status, variant, /*factored=*/0, stream, /*gamma_k_full=*/nullptr,
                                 /*after_prepare=*/true);
}

// Full fusion: one launch, no prepared-K tensor; the kernel normalises and rotates every K tile after it lands
// (the reference's `launch_attention(mode='full')`, src/e1_rope_publication_v1.py:667-677 with FUSE_K :633-634).
// The reference keeps this form as an ablation - every query tile repeats the K transform - and so does this
// library: it runs on the baseline kernel only.  Results equal those of kf_optimized_attention with variant 1
// bit for bit (same rounding points, same loop).
int kf_attention_full(const void* q, const void* k, const void* v, const void* gamma_q, const void* gamma_k,
                      const void* cos_table, const void* sin_table, void* out, int B, int Hq, int Hkv, int S, int D,
                      int dtype, int causal, int hf_norm, float eps, float scale, int64_t q_sb, int64_t q_sh,
                      int64_t q_ss, int64_t k_sb, int64_t k_sh, int64_t k_ss, int64_t v_sb, int64_t v_sh, int64_t v_ss,
                      int64_t o_sb, int64_t o_sh, int64_t o_ss, int* status, void* stream) {
    if (!gamma_q || !gamma_k) return fail(KF_EINVAL, "gamma_q and gamma_k must not be NULL");
    return attention_impl(q, k, v, gamma_q, cos_table, sin_table, out, B, Hq, Hkv, S, D, dtype, causal, hf_norm,
                          /*fuse_q=*/1, eps, scale, q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_sb, o_sh,
                          o_ss, status, /*variant=*/1, /*factored=*/0, stream, gamma_k);
}

// Factored no-RoPE form of the operator (the reference's `launch_factored_attention`,
// src/e1_qk_publication_v3.py:638-650): KN = r(k * inv_k * gamma_k * gamma_q) is written to `kn`, the raw
// query feeds the score product and each row's scores are scaled by its inverse RMS, which stays on chip
// (the reference stores it in a separate FP32 tensor).
int kf_factored_attention(const void* q, const void* k, const void* v, const void* gamma_q, const void* gamma_k,
                          void* kn, void* out, int B, int Hq, int Hkv, int S, int D, int dtype, int causal, float eps,
                          float scale, int64_t q_sb, int64_t q_sh, int64_t q_ss, int64_t k_sb, int64_t k_sh,
                          int64_t k_ss, int64_t v_sb, int64_t v_sh, int64_t v_ss, int64_t n_sb, int64_t n_sh,
                          int64_t n_ss, int64_t o_sb, int64_t o_sh, int64_t o_ss, int* status, int variant,
                          void* stream) {
    if (!gamma_q || !gamma_k) return fail(KF_EINVAL, "gamma_q and gamma_k must not be NULL");
    if (int r = prepare_impl(k, kn, gamma_k, gamma_q, nullptr, nullptr, B, Hkv, S, D, dtype, /*hf_norm=*/0, eps, k_sb,
                             k_sh, k_ss, n_sb, n_sh, n_ss, stream))
        return r;
    return attention_impl(q, kn, v, gamma_q, nullptr, nullptr, out, B, Hq, Hkv, S, D, dtype, causal, /*hf_norm=*/0,
                          /*fuse_q=*/1, eps, scale, q_sb, q_sh, q_ss, n_sb, n_sh, n_ss, v_sb, v_sh, v_ss, o_sb, o_sh,
                          o_ss, status, variant, /*factored=*/1, stream, /*gamma_k_full=*/nullptr, /*after_prepare=*/true);
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Allocation-free variant of the whole operator.
//
// Some callers cannot allocate device memory at the moment they need the
// operator: code that runs under a framework which owns the whole device heap
// and hands out no raw allocations, plugins invoked from inside a region where
// cudaMalloc is forbidden (it synchronises the device and is illegal while a
// stream is being captured), or real-time serving loops that must not touch
// the allocator on the request path.  For them the prepared-K scratch lives in
// the fixed array below, which is part of the library image: every GPU that
// loads the library reserves kStaticScratchBytes for it until the process
// exits.
constexpr size_t kStaticScratchBytes = 32u << 20;  // 32 MiB: B*Hkv*S*D*2 bytes must fit
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {
// The array's name is only a host-side handle; kernels need its device address,
// which differs per device and is looked up once per device (with that device
// current) through cudaGetSymbolAddress.
std::atomic<void*> g_scratch_addr[64];  // (atomic: two host threads may make a device's first call at once)

int static_scratch_for_current_device(void** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail(KF_ECUDA, "cudaGetDevice failed");
    if (dev < 0 || dev >= 64) return fail(KF_ECUDA, "device ordinal %d out of range", dev);
    void* p = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail(KF_ECUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        g_scratch_addr[dev].store(p, std::memory_order_release);  // (a concurrent first call stores the same address)
    }
    *out = p;
    return KF_OK;
}
}  // namespace

extern "C" {

size_t kf_static_scratch_bytes(void) { return kStaticScratchBytes; }

int kf_optimized_attention_static(const void* q, const void* k, const void* v, const void* gamma_q,
                                  const void* gamma_k, const void* cos_table, const void* sin_table, void* out,
                                  int B, int Hq, int Hkv, int S, int D, int dtype, int causal, int hf_norm,
                                  float eps, float scale, int64_t q_sb, int64_t q_sh, int64_t q_ss, int64_t k_sb,
                                  int64_t k_sh, int64_t k_ss, int64_t v_sb, int64_t v_sh, int64_t v_ss,
                                  int64_t o_sb, int64_t o_sh, int64_t o_ss, int* status, void* stream) {
    if (int r = check_common(B, Hq, S, D, dtype)) return r;
    if (Hkv < 1 || Hq % Hkv != 0) return fail(KF_EINVAL, "Hq (%d) must be a positive multiple of Hkv (%d)", Hq, Hkv);
    const unsigned long long need = 2ull * (unsigned long long)B * Hkv * S * D;
    if (need > kStaticScratchBytes)
        return fail(KF_EINVAL,
                    "prepared K needs %llu bytes (B*Hkv*S*D*2) but the built-in scratch holds %llu; "
                    "use kf_prepare_rows + kf_attention_fwd with a caller-allocated buffer",
                    need, (unsigned long long)kStaticScratchBytes);
    void* kn = nullptr;
    if (int r = static_scratch_for_current_device(&kn)) return r;
    // prepared K is laid out contiguously [B, Hkv, S, D] at the start of the scratch;
    // every row the attention kernel reads is rewritten by this call, so nothing
    // needs clearing between calls.
    const int64_t n_ss = D, n_sh = (int64_t)S * D, n_sb = (int64_t)Hkv * S * D;
    if (int r = kf_prepare_rows(k, kn, gamma_k, cos_table, sin_table, B, Hkv, S, D, dtype, hf_norm, eps, k_sb, k_sh,
                                k_ss, n_sb, n_sh, n_ss, stream))
        return r;
    return kf_attention_fwd(q, kn, v, gamma_q, cos_table, sin_table, out, B, Hq, Hkv, S, D, dtype, causal, hf_norm,
                            /*fuse_q=*/1, eps, scale, q_sb, q_sh, q_ss, n_sb, n_sh, n_ss, v_sb, v_sh, v_ss, o_sb,
                            o_sh, o_ss, status, /*variant=*/0, stream);
}

}  // extern "C"
