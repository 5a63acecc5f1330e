// The rounding contract of the row transform (RMSNorm -> gamma -> split-half
// RoPE), shared by the K-prepare kernel and the attention kernel's Q prologue.
//
// Follows the reference's `_rows` (src/e1_rope_publication_v1.py:551-582):
//   inv = rsqrt(sum(x^2)/D + eps)                        (fp32)
//   hf:      y = r(r(x*inv) * gamma)        legacy:  y = r(x*inv*gamma)
//   rope:    out_j = r(r(y_j*cos_j) - r(p_j*sin_j))  for j <  D/2, p_j = y_{j+D/2}
//            out_j = r(r(y_j*cos_j) + r(p_j*sin_j))  for j >= D/2, p_j = y_{j-D/2}
// where r(.) rounds to the 16-bit storage type (nearest even) and cos_j/sin_j
// are the table entries of the OUTPUT column j.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace kf {

template <typename T> struct Num;
template <> struct Num<__nv_bfloat16> {
    static constexpr uint32_t kFmt = 1;  // UMMA 16-bit format code
    __device__ static __forceinline__ float2 unpack(uint32_t u) {
        // bf16 -> fp32 is a 16-bit shift
        return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
    }
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __device__ static __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};
template <> struct Num<__half> {
    static constexpr uint32_t kFmt = 0;
    __device__ static __forceinline__ float2 unpack(uint32_t u) {
        return __half22float2(*reinterpret_cast<__half2*>(&u));
    }
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    __device__ static __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
};

// 8 packed 16-bit values (one 16-byte chunk) <-> 8 floats
template <typename T> __device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    float2 a = Num<T>::unpack(u.x), b = Num<T>::unpack(u.y), c = Num<T>::unpack(u.z), d = Num<T>::unpack(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
template <typename T> __device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(Num<T>::pack(f[0], f[1]), Num<T>::pack(f[2], f[3]), Num<T>::pack(f[4], f[5]),
                      Num<T>::pack(f[6], f[7]));
}
__device__ __forceinline__ float sumsq8(const float (&f)[8], float acc) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fmaf(f[i], f[i], acc);
    return acc;
}

// Normalise one element (no rotation yet).
template <typename T> __device__ __forceinline__ float norm1(float x, float inv, float g, bool hf) {
    if (hf) return Num<T>::round(__fmul_rn(Num<T>::round(__fmul_rn(x, inv)), g));
    return Num<T>::round(__fmul_rn(__fmul_rn(x, inv), g));
}

// Transform the chunk pair (lo: columns j..j+7 < D/2, hi: columns j+D/2..).
// g*/c*/s* are the gamma and table chunks at the same columns.  In place.
template <typename T>
__device__ __forceinline__ void transform_pair(float (&lo)[8], float (&hi)[8], float inv, const float (&glo)[8],
                                               const float (&ghi)[8], const float (&clo)[8], const float (&chi)[8],
                                               const float (&slo)[8], const float (&shi)[8], bool hf, bool rope) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float a = norm1<T>(lo[i], inv, glo[i], hf);
        float b = norm1<T>(hi[i], inv, ghi[i], hf);
        if (rope) {
            float pa = Num<T>::round(__fmul_rn(a, clo[i]));
            float ra = Num<T>::round(__fmul_rn(b, slo[i]));
            float pb = Num<T>::round(__fmul_rn(b, chi[i]));
            float rb = Num<T>::round(__fmul_rn(a, shi[i]));
            a = __fsub_rn(pa, ra);  // rounded to T by the final pack
            b = __fadd_rn(pb, rb);
        }
        lo[i] = a;
        hi[i] = b;
    }
}

}  // namespace kf
