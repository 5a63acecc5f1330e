// The rounding contract of the row transform (RMSNorm -> gamma -> split-half
// RoPE), shared by the row-prepare kernel and the attention kernel's Q prologue.
//
// Follows the reference's `_rows` (src/e1_rope_publication_v1.py:551-582):
//   inv = rsqrt(sum(x^2)/D + eps)                        (fp32)
//   hf:      y = r(r(x*inv) * gamma)        legacy:  y = r(x*inv*gamma)
//   rope:    out_j = r(y_j*cos_j - r(p_j*sin_j))  for j <  D/2, p_j = y_{j+D/2}
//            out_j = r(y_j*cos_j + r(p_j*sin_j))  for j >= D/2, p_j = y_{j-D/2}
// where r(.) rounds to the 16-bit storage type (nearest even) and cos_j/sin_j
// are the table entries of the OUTPUT column j.  The source spells the rotation
// as r(r(y*c) -+ r(p*s)), but the reference's compiled kernels contract the
// primary product into a fused multiply-add: on B200 the Triton arm's prepared K
// equals the form above bit for bit (up to the summation order of the row's sum of
// squares, ~1e-5 of the elements) and differs from the uncontracted spelling in
// 12-23 % of the elements.  The contracted form is what this code reproduces.
//
// Every r(a op b) whose operands are already 16-bit values is ONE packed
// 16-bit instruction (mul / fma .rn on bf16x2 / f16x2 round the exact result
// once), so the contract costs about five instructions per element instead
// of a convert round trip at every rounding point.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>

namespace kf {

template <typename T> struct Num;
template <> struct Num<__nv_bfloat16> {
    static constexpr uint32_t kFmt = 1;  // UMMA 16-bit format code
    __device__ static __forceinline__ float2 unpack(uint32_t u) {
        return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
    }
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        uint32_t r;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    }
    __device__ static __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
    __device__ static __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
    __device__ static __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
    __device__ static __forceinline__ uint32_t fma2(uint32_t a, uint32_t b, uint32_t c) {  // r(a*b + c)
        uint32_t r;
        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
        return r;
    }
};
template <> struct Num<__half> {
    static constexpr uint32_t kFmt = 0;
    __device__ static __forceinline__ float2 unpack(uint32_t u) {
        return __half22float2(*reinterpret_cast<__half2*>(&u));
    }
    __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
        uint32_t r;
        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
        return r;
    }
    __device__ static __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
    __device__ static __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
    __device__ static __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) {
        uint32_t r;
        asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
        return r;
    }
    __device__ static __forceinline__ uint32_t fma2(uint32_t a, uint32_t b, uint32_t c) {  // r(a*b + c)
        uint32_t r;
        asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
        return r;
    }
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
// sum of squares of the 8 values of a chunk, accumulated into acc
template <typename T> __device__ __forceinline__ float sumsq_chunk(const uint4& u, float acc) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = Num<T>::unpack(w[i]);
        acc = fmaf(f.x, f.x, acc);
        acc = fmaf(f.y, f.y, acc);
    }
    return acc;
}

// Normalise two packed elements: hf -> r(r(x*inv)*g); legacy -> r(x*inv*g).
template <typename T> __device__ __forceinline__ uint32_t norm2(uint32_t x, float inv, uint32_t g, bool hf) {
    const float2 f = Num<T>::unpack(x);
    if (hf) return Num<T>::mul2(Num<T>::pack(__fmul_rn(f.x, inv), __fmul_rn(f.y, inv)), g);
    const float2 gf = Num<T>::unpack(g);
    return Num<T>::pack(__fmul_rn(__fmul_rn(f.x, inv), gf.x), __fmul_rn(__fmul_rn(f.y, inv), gf.y));
}

// r(((x * inv) * g) * g2) for the 8 values of a chunk: the fp32 product chain of the reference's factored
// K-prepare (src/e1_qk_publication_v3.py:609), rounded once.
template <typename T>
__device__ __forceinline__ void scale_chunk2(uint4& x, float inv, const uint4& g, const uint4& g2) {
    uint32_t* w = reinterpret_cast<uint32_t*>(&x);
    const uint32_t* a = reinterpret_cast<const uint32_t*>(&g);
    const uint32_t* b = reinterpret_cast<const uint32_t*>(&g2);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = Num<T>::unpack(w[i]), ga = Num<T>::unpack(a[i]), gb = Num<T>::unpack(b[i]);
        w[i] = Num<T>::pack(__fmul_rn(__fmul_rn(__fmul_rn(f.x, inv), ga.x), gb.x),
                            __fmul_rn(__fmul_rn(__fmul_rn(f.y, inv), ga.y), gb.y));
    }
}

// Transform the chunk pair (lo: columns j..j+7 < D/2, hi: columns j+D/2..) in
// place.  g*/c*/s* are the gamma and table chunks at the same columns.
template <typename T>
__device__ __forceinline__ void transform_pair(uint4& lo, uint4& hi, float inv, const uint4& glo, const uint4& ghi,
                                               const uint4& clo, const uint4& chi, const uint4& slo,
                                               const uint4& shi, bool hf, bool rope) {
    uint32_t* l = reinterpret_cast<uint32_t*>(&lo);
    uint32_t* h = reinterpret_cast<uint32_t*>(&hi);
    const uint32_t* gl = reinterpret_cast<const uint32_t*>(&glo);
    const uint32_t* gh = reinterpret_cast<const uint32_t*>(&ghi);
    const uint32_t* cl = reinterpret_cast<const uint32_t*>(&clo);
    const uint32_t* ch = reinterpret_cast<const uint32_t*>(&chi);
    const uint32_t* sl = reinterpret_cast<const uint32_t*>(&slo);
    const uint32_t* sh = reinterpret_cast<const uint32_t*>(&shi);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t ya = norm2<T>(l[i], inv, gl[i], hf);
        const uint32_t yb = norm2<T>(h[i], inv, gh[i], hf);
        if (rope) {
            // (flipping both sign bits negates the rounded product exactly)
            l[i] = Num<T>::fma2(ya, cl[i], Num<T>::mul2(yb, sl[i]) ^ 0x80008000u);
            h[i] = Num<T>::fma2(yb, ch[i], Num<T>::mul2(ya, sh[i]));
        } else {
            l[i] = ya;
            h[i] = yb;
        }
    }
}

}  // namespace kf
