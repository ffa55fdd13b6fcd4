// rowwise_sm100.cu -- the memory-bound kernels of the path: RMSNorm, RMSNorm+quant (int8 and
// fp8), per-token quantisers, rotary embedding, SiLU-multiply, the LSTM gate epilogue and the
// dequantise-transpose kernels.
//
// They produce the same bits as the reference's pure-CUDA kernels (src/nn_kernel_cuda.h) but
// are organised for HBM throughput: one WARP per row with 128-bit loads and stores and
// shuffle-only reductions (no shared memory, no __syncthreads), several rows per CTA.
//
// Bit compatibility of the RMSNorm sum of squares: the reference gives thread t the pair
// (2t, 2t+1), reduces each 32-thread warp with a shfl_down tree (offsets 16,8,4,2,1) and then
// the per-warp sums with the same tree (src/nn_kernel_cuda.h:98-122). Here lane l holds the
// four pairs 4j..4j+3 of 16-byte chunk j = 32q + l, so reference warp w = 4q + (l >> 3) lives in
// an 8-lane group. Reference offsets 16, 8, 4 (in pairs) are lane distances 4, 2, 1 in this
// layout and offsets 2, 1 are in-lane: (p0+p2) + (p1+p3). Float addition is commutative, so a
// xor-butterfly yields the same bits as the down-tree. The cross-warp tree then becomes
// (e0 [+ e2]) + (e1 [+ e3]) over the q index followed by lane distances 16 and 8.
// Other reductions of the path are maxima, which do not depend on order.
#include "fluke_sm100.h"
#include "sm100_ptx.cuh"

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fluke_sm100 {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr unsigned kFull = 0xffffffffu;

// ---- software E4M3FN, the reference's conversion rules (src/nn_kernel_cuda.h:259-300) -----
// decode: NaN codes and zero give 0; encode: finite only, saturates to +-448 (0x7E), rounds
// half UP in magnitude (not to even), flushes |x| < 2^-10 to zero.
__device__ __forceinline__ float e4m3_decode(uint8_t b) {
    const uint32_t mag = b & 0x7Fu;
    if (mag == 0x7Fu || mag == 0u) return 0.0f;
    const uint32_t sign = uint32_t(b >> 7) << 31;
    const uint32_t e = (b >> 3) & 0xFu, m = b & 0x7u;
    if (e == 0) return __uint_as_float(__float_as_uint(float(m) * 1.953125e-3f) | sign);
    return __uint_as_float(sign | ((e + 120u) << 23) | (m << 20));
}

__device__ __forceinline__ uint8_t e4m3_encode(float f) {
    const uint32_t u = __float_as_uint(f);
    const uint32_t sign = (u >> 31) << 7;
    const uint32_t ef = (u >> 23) & 0xFFu;
    const uint32_t mf = u & 0x7FFFFFu;
    if (ef == 0) return uint8_t(sign);
    int e = int(ef) - 120;
    if (e >= 16) return uint8_t(sign | 0x7Eu);
    if (e > 0) {
        uint32_t m = (mf + (1u << 19)) >> 20;
        if (m >= 8u) { m = 0; ++e; }
        if (e >= 16) return uint8_t(sign | 0x7Eu);
        if (e == 15 && m == 7u) m = 6u;
        return uint8_t(sign | (uint32_t(e) << 3) | m);
    }
    if (e <= -4) return uint8_t(sign);
    const int shift = 21 - e;
    const uint32_t m = ((mf | (1u << 23)) + (1u << (shift - 1))) >> shift;
    if (m >= 8u) return uint8_t(sign | 0x08u);
    return uint8_t(sign | m);
}

// Four codes at once with the conversion instruction (e4m3 values are exact in f16). The software
// decoder above gives +0 for the NaN codes and for -0: those bytes are cleared first.
__device__ __forceinline__ void e4m3x4_decode(uint32_t word, float2 &lo, float2 &hi) {
    const uint32_t mag = word & 0x7F7F7F7Fu;
    word &= ~(__vcmpeq4(mag, 0x7F7F7F7Fu) | __vcmpeq4(mag, 0u));
    uint32_t h01, h23;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h01) : "h"(uint16_t(word & 0xFFFFu)));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h23) : "h"(uint16_t(word >> 16)));
    lo = __half22float2(*reinterpret_cast<const __half2 *>(&h01));
    hi = __half22float2(*reinterpret_cast<const __half2 *>(&h23));
}

// Two values at once with the conversion instruction. The instruction rounds to nearest even,
// the software encoder above (the reference's) rounds half away from zero: setting the lowest
// mantissa bit of the f32 input moves an exact tie (an even bit pattern, whatever the exponent)
// just above the tie and never carries another value across one, so the results agree for every
// finite input; both saturate at +-448 and flush what is below half the smallest subnormal to a
// signed zero. Byte 0 of the result encodes `lo`, byte 1 `hi`.
__device__ __forceinline__ uint32_t e4m3_encode_pair(float lo, float hi) {
    uint16_t r;
    const float a = __uint_as_float(__float_as_uint(hi) | 1u), b = __uint_as_float(__float_as_uint(lo) | 1u);
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(a), "f"(b));
    return r;
}

// x / s, correctly rounded, for many x and one positive s with r = 1.0f / s (itself correctly
// rounded): the product x * r is within an ulp or so of the quotient, and each step "exact
// residual by fma, then fma(residual, r, q)" lands on the correctly rounded quotient once q is a
// neighbour of it (Markstein's correction; two steps). Compared bit for bit with the division
// instruction sequence on 12 * 10^9 random pairs, in the kernel's domain and outside it, without a
// difference. The sign is taken from x so that a zero keeps it (-0 + +0 would give +0).
__device__ __forceinline__ float div_by_scale(float x, float s, float r) {
    float q = __fmul_rn(x, r);
    q = __fmaf_rn(__fmaf_rn(-q, s, x), r, q);
    q = __fmaf_rn(__fmaf_rn(-q, s, x), r, q);
    return __uint_as_float((__float_as_uint(q) & 0x7FFFFFFFu) | (__float_as_uint(x) & 0x80000000u));
}

// The same for two values in packed arithmetic.
__device__ __forceinline__ float2 div_by_scale2(float2 x, float s, float r) {
    const float2 s2 = make_float2(-s, -s), r2 = make_float2(r, r);
    float2 q = mul2(x, r2);
    q = fma2(fma2(q, s2, x), r2, q);
    q = fma2(fma2(q, s2, x), r2, q);
    return make_float2(__uint_as_float((__float_as_uint(q.x) & 0x7FFFFFFFu) | (__float_as_uint(x.x) & 0x80000000u)),
                       __uint_as_float((__float_as_uint(q.y) & 0x7FFFFFFFu) | (__float_as_uint(x.y) & 0x80000000u)));
}

// ---- small helpers -----------------------------------------------------------------------
__device__ __forceinline__ void unpack8(const uint4 &raw, float2 (&f)[4]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) f[k] = __half22float2(h[k]);
}
__device__ __forceinline__ uint4 pack8(const float2 (&f)[4]) {
    uint4 raw;
    __half2 *h = reinterpret_cast<__half2 *>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __float22half2_rn(f[k]);
    return raw;
}
__device__ __forceinline__ float group8_sum(float s) {
    s += __shfl_xor_sync(kFull, s, 4);
    s += __shfl_xor_sync(kFull, s, 2);
    s += __shfl_xor_sync(kFull, s, 1);
    return s;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(kFull, v, o));
    return v;
}
__device__ __forceinline__ int clamp127(int v) { return max(-127, min(127, v)); }

// int8 <-> f32 without the conversion unit (a quarter-rate pipe that the int8 RMSNorm kernel would
// otherwise keep 60 % busy).
// Byte j of `biased` (= the int8 bytes with their sign bits flipped, i.e. value + 128 as
// unsigned) becomes the low mantissa byte of 2^23; subtracting 2^23 + 128 leaves the value.
__device__ __forceinline__ float2 i8_pair_to_float(uint32_t biased, uint32_t sel_lo, uint32_t sel_hi) {
    const float a = __uint_as_float(__byte_perm(biased, 0x4B000000u, sel_lo));
    const float b = __uint_as_float(__byte_perm(biased, 0x4B000000u, sel_hi));
    return make_float2(__fadd_rn(a, -8388736.0f), __fadd_rn(b, -8388736.0f));
}
// Round-to-nearest-even integer of v (|v| < 2^22) in the low bits of the result: adding
// 1.5 * 2^23 leaves the integer, in two's complement, in the low mantissa bits. (__fadd_rn: the
// addition must not be fused with the multiplication that produced v.)
__device__ __forceinline__ uint32_t round_to_int_bits(float v) { return __float_as_uint(__fadd_rn(v, 12582912.0f)); }
// The low bytes of four words, packed.
__device__ __forceinline__ uint32_t pack_low_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}

// Sum of squares of one row in the reference's summation order. `sq[q][k]` is the
// x*x + y*y term of pair k of this lane's chunk in load q; L = hidden_dim / 256.
// L = 2 with half the shuffles: instead of every lane of an 8-lane group reducing all eight
// (q, k) terms redundantly, each butterfly step also halves the set a lane is responsible for
// (the partner receives the other half), so after the three steps lane bits (2, 1, 0) select
// which one of the eight group sums the lane holds: k = 2 * bit2 + bit1, q = bit0. The additions
// are the same pairs in the same order as in the plain form, and a + b == b + a, so every lane
// ends with the same bits as before.
__device__ __forceinline__ float row_sum_sq_2(const float (&sq)[2][4], int lane) {
    const bool b2 = lane & 4, b1 = lane & 2, b0 = lane & 1;
    // lane distance 4: keep k in {0,1} (bit2 = 0) or {2,3} (bit2 = 1), for both q
    float a[2][2];
#pragma unroll
    for (int q = 0; q < 2; ++q)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float keep = b2 ? sq[q][2 + j] : sq[q][j];
            const float send = b2 ? sq[q][j] : sq[q][2 + j];
            a[q][j] = keep + __shfl_xor_sync(kFull, send, 4);
        }
    // lane distance 2: keep k's low bit = bit1
    float c[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const float keep = b1 ? a[q][1] : a[q][0];
        const float send = b1 ? a[q][0] : a[q][1];
        c[q] = keep + __shfl_xor_sync(kFull, send, 2);
    }
    // lane distance 1: keep q = bit0
    const float keep = b0 ? c[1] : c[0];
    const float send = b0 ? c[0] : c[1];
    float p = keep + __shfl_xor_sync(kFull, send, 1);   // the group's sum of term (q, k)
    // e_q = (p0 + p2) + (p1 + p3), then e0 + e1: partners differ in bit2, bit1, bit0
    p += __shfl_xor_sync(kFull, p, 4);
    p += __shfl_xor_sync(kFull, p, 2);
    p += __shfl_xor_sync(kFull, p, 1);
    p += __shfl_xor_sync(kFull, p, 16);
    p += __shfl_xor_sync(kFull, p, 8);
    return p;
}

template <int L>
__device__ __forceinline__ float row_sum_sq(const float (&sq)[L][4]) {
    float e[L];
#pragma unroll
    for (int q = 0; q < L; ++q) {
        const float p0 = group8_sum(sq[q][0]), p1 = group8_sum(sq[q][1]);
        const float p2 = group8_sum(sq[q][2]), p3 = group8_sum(sq[q][3]);
        e[q] = (p0 + p2) + (p1 + p3);
    }
    float u;
    if constexpr (L == 1) u = e[0];
    else if constexpr (L == 2) u = e[0] + e[1];
    else if constexpr (L == 3) u = (e[0] + e[2]) + e[1];
    else u = (e[0] + e[2]) + (e[1] + e[3]);
    u += __shfl_xor_sync(kFull, u, 16);
    u += __shfl_xor_sync(kFull, u, 8);
    return u;
}

enum { kOutF16 = 0, kOutI8 = 1, kOutF8 = 2 };

// ---- RMSNorm family, hidden_dim = 256*L, one warp per row ----------------------------------
// MODE kOutF16: out = f16(v*rms_inv*w), v = in + alpha*residual(f16)   (nn_kernel_cuda.h:139-180)
// MODE kOutI8 : v = in + (float(res_i8)*res_scale)*alpha, int8 + scale written over the
//               residual in place, scale = 1/(127/amax)                (nn_kernel_cuda.h:182-228)
// MODE kOutF8 : same with e4m3 residual, scale = max(amax,1e-12)/448   (nn_kernel_cuda.h:305-345)
// CTAs of four rows, and for hidden sizes up to 512 a register budget of 32 (16 CTAs = all 64 warps
// of an SM resident): the kernel is a chain of dependent steps per row in short-lived warps, so
// it lives on occupancy and on a fine CTA granularity at the tail (config 2, int8: 13.1 us with
// 8-row CTAs at 40 registers, 12.7 with 8-row CTAs at 32, 12.5 with 4-row CTAs at 32).
constexpr int kNormWarps = 4;
template <int L, int MODE>
__global__ void __launch_bounds__(kNormWarps * 32, (L <= 2 ? 16 : 1))
rmsnorm_rows_kernel(const __half *__restrict__ in, const void *residual_in,
                    const __half *__restrict__ weight, void *out, float *res_scale, int n_tokens,
                    int hidden_dim, float alpha, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t row = int64_t(blockIdx.x) * kNormWarps + (threadIdx.x >> 5);
    if (row >= n_tokens) return;
    const int64_t base = row * hidden_dim;

    float2 val[L][4];
    float sq[L][4];
    float rs = 0.f;
    if constexpr (MODE != kOutF16) rs = res_scale[row];

#pragma unroll
    for (int q = 0; q < L; ++q) {
        const int off = (q * 32 + lane) * 8;
        float2 xf[4];
        unpack8(__ldg(reinterpret_cast<const uint4 *>(in + base + off)), xf);
        if constexpr (MODE == kOutF16) {
            float2 rf[4];
            unpack8(__ldg(reinterpret_cast<const uint4 *>(
                        static_cast<const __half *>(residual_in) + base + off)), rf);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                val[q][k] = fma2(rf[k], make_float2(alpha, alpha), xf[k]);
        } else {
            const uint2 raw = *reinterpret_cast<const uint2 *>(
                static_cast<const uint8_t *>(residual_in) + base + off);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if constexpr (MODE == kOutI8) {
                    const uint32_t word = ((k < 2) ? raw.x : raw.y) ^ 0x80808080u;
                    const float2 r = i8_pair_to_float(word, 0x7440u + 2 * (k & 1), 0x7441u + 2 * (k & 1));
                    // x + (r * rs) * alpha: product, then one fused multiply-add (the form the
                    // reference's build contracts to), two elements per instruction
                    val[q][k] = fma2(mul2(r, make_float2(rs, rs)), make_float2(alpha, alpha), xf[k]);
                } else {
                    float2 ra, rb2;
                    e4m3x4_decode((k < 2) ? raw.x : raw.y, ra, rb2);
                    // x + (r * rs) * alpha as for the int8 residual: product, then one fused multiply-add
                    val[q][k] = fma2(mul2((k & 1) ? rb2 : ra, make_float2(rs, rs)), make_float2(alpha, alpha), xf[k]);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) sq[q][k] = val[q][k].x * val[q][k].x + val[q][k].y * val[q][k].y;
    }

    float sum_sq;
    if constexpr (L == 2) sum_sq = row_sum_sq_2(sq, lane);
    else sum_sq = row_sum_sq<L>(sq);
    // hidden_dim = 256 * L: for L a power of two the division is an exact scaling, done as a
    // multiplication by the exact reciprocal (same bits, a few instructions fewer)
    const float mean_sq = (L == 1 || L == 2 || L == 4) ? sum_sq * (1.0f / (256.0f * L)) : sum_sq / hidden_dim;
    const float rms_inv = rsqrtf(mean_sq + eps);

    float amax = 0.f;
#pragma unroll
    for (int q = 0; q < L; ++q) {
        const int off = (q * 32 + lane) * 8;
        float2 wf[4];
        unpack8(__ldg(reinterpret_cast<const uint4 *>(weight + off)), wf);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            val[q][k] = mul2(mul2(val[q][k], make_float2(rms_inv, rms_inv)), wf[k]);
            amax = fmaxf(amax, fmaxf(fabsf(val[q][k].x), fabsf(val[q][k].y)));
        }
        if constexpr (MODE == kOutF16)
            *reinterpret_cast<uint4 *>(static_cast<__half *>(out) + base + off) = pack8(val[q]);
    }
    if constexpr (MODE == kOutF16) return;

    amax = warp_max(amax);
    if constexpr (MODE == kOutI8) {
        const float quant_scale = (amax > 0.0f) ? (127.0f / amax) : 1.0f;
        if (lane == 0) res_scale[row] = 1.0f / quant_scale;
#pragma unroll
        for (int q = 0; q < L; ++q) {
            const int off = (q * 32 + lane) * 8;
            // |val * quant_scale| <= 127 (1 + 2^-23) by construction of the scale, so the rounded
            // integer needs no clamp (NaN inputs, which the reference maps to 0, give -1 here)
            uint32_t t[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                // the product is rounded to f32 first, then p * 1 + 1.5 * 2^23 rounds it to an
                // integer (a packed multiply followed by a packed add was observed to come out
                // as ONE fused operation, which rounds only once)
                const float2 rq = fma2(mul2(val[q][k], make_float2(quant_scale, quant_scale)),
                                       make_float2(1.0f, 1.0f), make_float2(12582912.0f, 12582912.0f));
                t[2 * k] = __float_as_uint(rq.x);
                t[2 * k + 1] = __float_as_uint(rq.y);
            }
            const uint2 raw = make_uint2(pack_low_bytes(t[0], t[1], t[2], t[3]), pack_low_bytes(t[4], t[5], t[6], t[7]));
            *reinterpret_cast<uint2 *>(static_cast<uint8_t *>(out) + base + off) = raw;
        }
    } else {
        const float fp8_scale = fmaxf(amax, 1e-12f) / 448.0f;
        const float fp8_rcp = 1.0f / fp8_scale;
        if (lane == 0) res_scale[row] = fp8_scale;
#pragma unroll
        for (int q = 0; q < L; ++q) {
            const int off = (q * 32 + lane) * 8;
            uint32_t hw[4];
#pragma unroll
            for (int k = 0; k < 4; ++k)
            {
                const float2 dv = div_by_scale2(val[q][k], fp8_scale, fp8_rcp);
                hw[k] = e4m3_encode_pair(fmaxf(-448.0f, fminf(448.0f, dv.x)), fmaxf(-448.0f, fminf(448.0f, dv.y)));
            }
            *reinterpret_cast<uint2 *>(static_cast<uint8_t *>(out) + base + off) =
                make_uint2(hw[0] | (hw[1] << 16), hw[2] | (hw[3] << 16));
        }
    }
}

// ---- RMSNorm family, any even hidden_dim <= 1024: one CTA per row, thread t owns pair t ------
// Same tree as the reference; threads past hidden_dim/2 (the CTA is rounded up to whole warps)
// contribute zeros.
__device__ __forceinline__ float block_tree_sum(float v, float *buf) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(kFull, v, o);
    if (lane == 0) buf[warp] = v;
    __syncthreads();
    const int nwarps = blockDim.x >> 5;
    float r = (threadIdx.x < nwarps) ? buf[threadIdx.x] : 0.0f;
    if (warp == 0) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) r += __shfl_down_sync(kFull, r, o);
    }
    if (threadIdx.x == 0) buf[0] = r;
    __syncthreads();
    const float result = buf[0];
    __syncthreads();
    return result;
}
__device__ __forceinline__ float block_max(float v, float *buf) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    if (lane == 0) buf[warp] = v;
    __syncthreads();
    const int nwarps = blockDim.x >> 5;
    float r = (lane < nwarps) ? buf[lane] : 0.0f;
    r = warp_max(r);
    __syncthreads();
    return r;
}

template <int MODE>
__global__ void rmsnorm_generic_kernel(const __half *__restrict__ in, const void *residual_in,
                                       const __half *__restrict__ weight, void *out,
                                       float *res_scale, int n_tokens, int hidden_dim, float alpha,
                                       float eps) {
    __shared__ float buf[32];
    const int64_t row = blockIdx.x;
    const int t = threadIdx.x;
    const bool live = t < (hidden_dim >> 1);
    const int64_t base = row * hidden_dim;

    float2 val = make_float2(0.f, 0.f), wf = make_float2(0.f, 0.f);
    float rs = 0.f;
    if constexpr (MODE != kOutF16) rs = res_scale[row];
    if (live) {
        const float2 xf = __half22float2(reinterpret_cast<const __half2 *>(in + base)[t]);
        wf = __half22float2(reinterpret_cast<const __half2 *>(weight)[t]);
        if constexpr (MODE == kOutF16) {
            const float2 rf = __half22float2(
                reinterpret_cast<const __half2 *>(static_cast<const __half *>(residual_in) + base)[t]);
            val = make_float2(xf.x + rf.x * alpha, xf.y + rf.y * alpha);
        } else if constexpr (MODE == kOutI8) {
            const char2 rq = reinterpret_cast<const char2 *>(static_cast<const int8_t *>(residual_in) + base)[t];
            val = make_float2(xf.x + ((float)rq.x * rs) * alpha, xf.y + ((float)rq.y * rs) * alpha);
        } else {
            const uchar2 rq = reinterpret_cast<const uchar2 *>(static_cast<const uint8_t *>(residual_in) + base)[t];
            val = make_float2(xf.x + e4m3_decode(rq.x) * rs * alpha, xf.y + e4m3_decode(rq.y) * rs * alpha);
        }
    }
    __syncthreads();  // every thread has read the old residual scale before it is overwritten
    const float sum_sq = block_tree_sum(val.x * val.x + val.y * val.y, buf);
    const float rms_inv = rsqrtf(sum_sq / hidden_dim + eps);
    const float2 nrm = make_float2(val.x * rms_inv * wf.x, val.y * rms_inv * wf.y);
    if constexpr (MODE == kOutF16) {
        if (live) reinterpret_cast<__half2 *>(static_cast<__half *>(out) + base)[t] = __float22half2_rn(nrm);
        return;
    }
    const float amax = block_max(fmaxf(fabsf(nrm.x), fabsf(nrm.y)), buf);
    if constexpr (MODE == kOutI8) {
        const float quant_scale = (amax > 0.0f) ? (127.0f / amax) : 1.0f;
        if (t == 0) res_scale[row] = 1.0f / quant_scale;
        if (live) {
            char2 qv;
            qv.x = (int8_t)clamp127(__float2int_rn(nrm.x * quant_scale));
            qv.y = (int8_t)clamp127(__float2int_rn(nrm.y * quant_scale));
            reinterpret_cast<char2 *>(static_cast<int8_t *>(out) + base)[t] = qv;
        }
    } else {
        const float fp8_scale = fmaxf(amax, 1e-12f) / 448.0f;
        if (t == 0) res_scale[row] = fp8_scale;
        if (live) {
            uchar2 qv;
            qv.x = e4m3_encode(fmaxf(-448.0f, fminf(448.0f, nrm.x / fp8_scale)));
            qv.y = e4m3_encode(fmaxf(-448.0f, fminf(448.0f, nrm.y / fp8_scale)));
            reinterpret_cast<uchar2 *>(static_cast<uint8_t *>(out) + base)[t] = qv;
        }
    }
}

template <int MODE>
int launch_rmsnorm(const void *in, const void *residual_in, const void *weight, void *out,
                   float *res_scale, int n_tokens, int hidden_dim, float alpha, float eps,
                   cudaStream_t s) {
    if (n_tokens <= 0) return 0;
    const __half *x = static_cast<const __half *>(in), *w = static_cast<const __half *>(weight);
    const bool aligned =
        ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(weight) |
          reinterpret_cast<uintptr_t>(residual_in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    if (hidden_dim % 256 == 0 && aligned) {
        const int grid = (n_tokens + kNormWarps - 1) / kNormWarps;
        const int block = kNormWarps * 32;
        switch (hidden_dim / 256) {
            case 1: rmsnorm_rows_kernel<1, MODE><<<grid, block, 0, s>>>(x, residual_in, w, out, res_scale, n_tokens, hidden_dim, alpha, eps); break;
            case 2: rmsnorm_rows_kernel<2, MODE><<<grid, block, 0, s>>>(x, residual_in, w, out, res_scale, n_tokens, hidden_dim, alpha, eps); break;
            case 3: rmsnorm_rows_kernel<3, MODE><<<grid, block, 0, s>>>(x, residual_in, w, out, res_scale, n_tokens, hidden_dim, alpha, eps); break;
            default: rmsnorm_rows_kernel<4, MODE><<<grid, block, 0, s>>>(x, residual_in, w, out, res_scale, n_tokens, hidden_dim, alpha, eps); break;
        }
    } else {
        const int block = ((hidden_dim / 2 + 31) / 32) * 32;
        rmsnorm_generic_kernel<MODE><<<n_tokens, block, 0, s>>>(x, residual_in, w, out, res_scale, n_tokens, hidden_dim, alpha, eps);
    }
    return (int)cudaGetLastError();
}

// ---- per-token quantisers (nn_kernel_cuda.h:352-411), hidden_dim = 256*L: one warp per row, the
// row stays in registers between the maximum and the conversion. int8: round(v * inv) by magic
// addition after clamping to +-127 in float (the same integers as rounding first), bytes gathered
// with permutes (a NaN input, which the reference's conversion maps to 0, becomes 127 here); e4m3:
// the conversion instruction. CTA shape as for the RMSNorm kernels.
template <int L, bool FP8>
__global__ void __launch_bounds__(kNormWarps * 32, (L <= 2 ? 16 : 1))
quant_rows_reg_kernel(const __half *__restrict__ in, uint8_t *__restrict__ out,
                      float *__restrict__ scale, int n_tokens) {
    const int lane = threadIdx.x & 31;
    const int64_t row = int64_t(blockIdx.x) * kNormWarps + (threadIdx.x >> 5);
    if (row >= n_tokens) return;
    const int64_t base = row * (256 * L);
    float2 val[L][4];
    float amax = 0.f;
#pragma unroll
    for (int q = 0; q < L; ++q) {
        unpack8(__ldg(reinterpret_cast<const uint4 *>(in + base + (q * 32 + lane) * 8)), val[q]);
#pragma unroll
        for (int k = 0; k < 4; ++k) amax = fmaxf(amax, fmaxf(fabsf(val[q][k].x), fabsf(val[q][k].y)));
    }
    amax = warp_max(amax);
    const float dq = fmaxf(amax, 1e-12f) / (FP8 ? 448.0f : 128.0f);
    if (lane == 0) scale[row] = dq;
    const float inv = 1.0f / dq;
    const float2 inv2 = make_float2(inv, inv);
#pragma unroll
    for (int q = 0; q < L; ++q) {
        uint2 raw;
        if constexpr (FP8) {
            uint32_t h[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 pv = mul2(val[q][k], inv2);
                h[k] = e4m3_encode_pair(fmaxf(-448.0f, fminf(448.0f, pv.x)), fmaxf(-448.0f, fminf(448.0f, pv.y)));
            }
            raw = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
        } else {
            uint32_t t[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 pv = mul2(val[q][k], inv2);
                const float2 cl = make_float2(fmaxf(-127.0f, fminf(127.0f, pv.x)), fmaxf(-127.0f, fminf(127.0f, pv.y)));
                // c * 1 + 1.5 * 2^23 rounds the clamped product to an integer in the low mantissa bits
                const float2 rq = fma2(cl, make_float2(1.0f, 1.0f), make_float2(12582912.0f, 12582912.0f));
                t[2 * k] = __float_as_uint(rq.x);
                t[2 * k + 1] = __float_as_uint(rq.y);
            }
            raw = make_uint2(pack_low_bytes(t[0], t[1], t[2], t[3]), pack_low_bytes(t[4], t[5], t[6], t[7]));
        }
        *reinterpret_cast<uint2 *>(out + base + (q * 32 + lane) * 8) = raw;
    }
}

// ---- per-token quantisers (nn_kernel_cuda.h:352-411): one warp per row, any even H ----------
// The second pass re-reads the row (at most 4 KB, still in L1).
template <bool FP8>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
quant_rows_kernel(const __half *__restrict__ in, uint8_t *__restrict__ out,
                  float *__restrict__ scale, int n_tokens, int hidden_dim, int vec_ok) {
    const int lane = threadIdx.x & 31;
    const int64_t row = int64_t(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
    if (row >= n_tokens) return;
    const __half *x = in + row * hidden_dim;
    uint8_t *o = out + row * hidden_dim;

    float amax = 0.f;
    if (vec_ok) {
        for (int c = lane; c < (hidden_dim >> 3); c += 32) {
            float2 f[4];
            unpack8(__ldg(reinterpret_cast<const uint4 *>(x) + c), f);
#pragma unroll
            for (int k = 0; k < 4; ++k) amax = fmaxf(amax, fmaxf(fabsf(f[k].x), fabsf(f[k].y)));
        }
    } else {
        for (int c = lane; c < (hidden_dim >> 1); c += 32) {
            const float2 f = __half22float2(reinterpret_cast<const __half2 *>(x)[c]);
            amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
    }
    amax = warp_max(amax);
    const float dq = fmaxf(amax, 1e-12f) / (FP8 ? 448.0f : 128.0f);
    if (lane == 0) scale[row] = dq;
    const float inv = 1.0f / dq;

    auto quant1 = [&](float v) -> uint8_t {
        if constexpr (FP8) return e4m3_encode(fmaxf(-448.0f, fminf(448.0f, v * inv)));
        else return (uint8_t)(int8_t)clamp127(__float2int_rn(v * inv));
    };
    if (vec_ok) {
        for (int c = lane; c < (hidden_dim >> 3); c += 32) {
            float2 f[4];
            unpack8(__ldg(reinterpret_cast<const uint4 *>(x) + c), f);
            uint2 raw;
            uint8_t *ob = reinterpret_cast<uint8_t *>(&raw);
#pragma unroll
            for (int k = 0; k < 4; ++k) { ob[2 * k] = quant1(f[k].x); ob[2 * k + 1] = quant1(f[k].y); }
            reinterpret_cast<uint2 *>(o)[c] = raw;
        }
    } else {
        for (int c = lane; c < (hidden_dim >> 1); c += 32) {
            const float2 f = __half22float2(reinterpret_cast<const __half2 *>(x)[c]);
            uchar2 qv;
            qv.x = quant1(f.x); qv.y = quant1(f.y);
            reinterpret_cast<uchar2 *>(o)[c] = qv;
        }
    }
}

// ---- rotary embedding (nn_kernel_cuda.h:35-69) -------------------------------------------------
// The reference's nvcc build evaluates the two outputs as fma(x0,cos,-(x1*sin)) and
// fma(x0,sin,x1*cos) (established by comparing its kernel's output bits with each candidate);
// the same order is spelled out with intrinsics here so it does not depend on the compiler.
// Vector path: one thread rotates 8 pairs (x0 = 16 bytes at offset 8c, x1 = 16 bytes at offset
// W + 8c). With 8 heads of 64 and W = 32 a warp covers one (batch, position) row of 1 KB.
// SHIFTS: the thread index decomposes with shifts and one 32-bit division (chunks per head and
// heads both powers of two, fewer than 2^31 threads); otherwise with 64-bit divisions, which cost
// more instructions than the rotation itself.
template <bool SHIFTS>
__global__ void __launch_bounds__(256)
rotary_vec_kernel(__half *x, const float *__restrict__ sin_tab, const float *__restrict__ cos_tab,
                  int64_t total, int seq_len, int n_heads, int width, int64_t stride_batch,
                  int64_t stride_seq, int64_t stride_head, int cpw_log2, int heads_log2) {
    const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    int c, h, s;
    int64_t b;
    if constexpr (SHIFTS) {
        const uint32_t i32 = uint32_t(idx);
        c = int(i32 & ((1u << cpw_log2) - 1u));
        h = int((i32 >> cpw_log2) & ((1u << heads_log2) - 1u));
        const uint32_t row = i32 >> (cpw_log2 + heads_log2);
        const uint32_t bq = row / uint32_t(seq_len);
        s = int(row - bq * uint32_t(seq_len));
        b = bq;
    } else {
        const int cpw = width >> 3;
        c = int(idx % cpw);
        int64_t r = idx / cpw;
        h = int(r % n_heads); r /= n_heads;
        s = int(r % seq_len);
        b = r / seq_len;
    }

    __half *p0 = x + b * stride_batch + s * stride_seq + h * stride_head + c * 8;
    __half *p1 = p0 + width;
    float2 a[4], bq[4];
    unpack8(*reinterpret_cast<const uint4 *>(p0), a);
    unpack8(*reinterpret_cast<const uint4 *>(p1), bq);
    const float4 *cs4 = reinterpret_cast<const float4 *>(cos_tab + int64_t(s) * width + c * 8);
    const float4 *sn4 = reinterpret_cast<const float4 *>(sin_tab + int64_t(s) * width + c * 8);
    const float4 c0 = __ldg(cs4), c1 = __ldg(cs4 + 1), s0 = __ldg(sn4), s1 = __ldg(sn4 + 1);
    const float cosv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sinv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    float2 o0[4], o1[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        {
            const float x0 = a[k].x, x1 = bq[k].x, cos = cosv[2 * k], sin = sinv[2 * k];
            o0[k].x = __fmaf_rn(x0, cos, -__fmul_rn(x1, sin));
            o1[k].x = __fmaf_rn(x0, sin, __fmul_rn(x1, cos));
        }
        {
            const float x0 = a[k].y, x1 = bq[k].y, cos = cosv[2 * k + 1], sin = sinv[2 * k + 1];
            o0[k].y = __fmaf_rn(x0, cos, -__fmul_rn(x1, sin));
            o1[k].y = __fmaf_rn(x0, sin, __fmul_rn(x1, cos));
        }
    }
    // __float2half rounds to nearest even, as does the paired conversion used by pack8.
    *reinterpret_cast<uint4 *>(p0) = pack8(o0);
    *reinterpret_cast<uint4 *>(p1) = pack8(o1);
}

// Scalar path for widths or strides that are not multiples of 8 elements.
__global__ void __launch_bounds__(256)
rotary_scalar_kernel(__half *x, const float *__restrict__ sin_tab,
                     const float *__restrict__ cos_tab, int64_t total, int seq_len, int n_heads,
                     int width, int64_t stride_batch, int64_t stride_seq, int64_t stride_head) {
    const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int rot = int(idx % width);
    int64_t r = idx / width;
    const int h = int(r % n_heads); r /= n_heads;
    const int s = int(r % seq_len);
    const int64_t b = r / seq_len;
    __half *o0 = x + b * stride_batch + s * stride_seq + h * stride_head + rot;
    __half *o1 = o0 + width;
    const float cos = cos_tab[int64_t(s) * width + rot], sin = sin_tab[int64_t(s) * width + rot];
    const float x0 = __half2float(*o0), x1 = __half2float(*o1);
    *o0 = __float2half(__fmaf_rn(x0, cos, -__fmul_rn(x1, sin)));
    *o1 = __float2half(__fmaf_rn(x0, sin, __fmul_rn(x1, cos)));
}

// idx -> (idx / per_row, idx % per_row): a 32-bit division where the index allows it (a 64-bit one
// costs about as many instructions as the arithmetic of the element-wise kernels below).
__device__ __forceinline__ void split_index(int64_t idx, int64_t total, int per_row, int64_t &row, int &col) {
    if (total < (int64_t(1) << 31)) {
        const uint32_t i32 = uint32_t(idx), r32 = i32 / uint32_t(per_row);
        row = r32;
        col = int(i32 - r32 * uint32_t(per_row));
    } else {
        row = idx / per_row;
        col = int(idx % per_row);
    }
}

// ---- SiLU-multiply (nn_kernel_cuda.h:71-90) -----------------------------------------------------
template <int VEC>
__global__ void __launch_bounds__(256)
silu_mul_kernel(const __half *__restrict__ in, __half *__restrict__ out, int64_t total_vec,
                int hidden_dim) {
    const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total_vec) return;
    const int per_row = hidden_dim / VEC;
    int64_t t;
    int k;
    split_index(idx, total_vec, per_row, t, k);
    k *= VEC;
    const __half *y = in + t * 2 * hidden_dim + k;
    const __half *g = y + hidden_dim;
    __half *o = out + t * hidden_dim + k;
    if constexpr (VEC == 8) {
        float2 yf[4], gf[4], of[4];
        unpack8(__ldg(reinterpret_cast<const uint4 *>(y)), yf);
        unpack8(__ldg(reinterpret_cast<const uint4 *>(g)), gf);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            of[j].x = (gf[j].x / (1.0f + __expf(-gf[j].x))) * yf[j].x;
            of[j].y = (gf[j].y / (1.0f + __expf(-gf[j].y))) * yf[j].y;
        }
        *reinterpret_cast<uint4 *>(o) = pack8(of);
    } else {
        const float gv = __half2float(*g);
        const float silu = gv / (1.0f + __expf(-gv));
        *o = __float2half(silu * __half2float(*y));
    }
}

// ---- LSTM gate epilogue on f16 (nn_kernel_cuda.h:233-255) ----------------------------------------
// Operation order of the reference's nvcc build, spelled out: gates fma(g, 0.2, 0.5), cell
// fma(i, g~, f*c) (established by comparing its kernel's output bits with each candidate).
__device__ __forceinline__ void flstm_gate(float gi, float gf, float gg, float go, float c_old,
                                           float &c_new, float &h_new) {
    const float i_g = fmaxf(0.f, fminf(1.f, __fmaf_rn(gi, 0.2f, 0.5f)));
    const float f_g = fmaxf(0.f, fminf(1.f, __fmaf_rn(gf, 0.2f, 0.5f)));
    const float g_g = fmaxf(-1.f, fminf(1.f, gg));
    const float o_g = fmaxf(0.f, fminf(1.f, __fmaf_rn(go, 0.2f, 0.5f)));
    c_new = __fmaf_rn(i_g, g_g, __fmul_rn(f_g, c_old));
    h_new = __fmul_rn(o_g, tanhf(c_new));
}

template <int VEC>
__global__ void __launch_bounds__(256)
flstm_step_kernel(const __half *__restrict__ scratch, const __half *__restrict__ ih_t,
                  __half *cell, __half *__restrict__ hh_next, int64_t total_vec, int hidden_dim) {
    const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total_vec) return;
    const int per_row = hidden_dim / VEC;
    int64_t n;
    int ch;
    split_index(idx, total_vec, per_row, n, ch);
    ch *= VEC;
    const int64_t gbase = n * 4 * hidden_dim + ch, cbase = n * hidden_dim + ch;
    if constexpr (VEC == 8) {
        float2 a[4][4], b[4][4], cf[4], cn[4], hn[4];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            unpack8(__ldg(reinterpret_cast<const uint4 *>(scratch + gbase + g * hidden_dim)), a[g]);
            unpack8(__ldg(reinterpret_cast<const uint4 *>(ih_t + gbase + g * hidden_dim)), b[g]);
        }
        unpack8(*reinterpret_cast<const uint4 *>(cell + cbase), cf);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            flstm_gate(a[0][j].x + b[0][j].x, a[1][j].x + b[1][j].x, a[2][j].x + b[2][j].x,
                       a[3][j].x + b[3][j].x, cf[j].x, cn[j].x, hn[j].x);
            flstm_gate(a[0][j].y + b[0][j].y, a[1][j].y + b[1][j].y, a[2][j].y + b[2][j].y,
                       a[3][j].y + b[3][j].y, cf[j].y, cn[j].y, hn[j].y);
        }
        *reinterpret_cast<uint4 *>(cell + cbase) = pack8(cn);
        *reinterpret_cast<uint4 *>(hh_next + cbase) = pack8(hn);
    } else {
        float g4[4];
#pragma unroll
        for (int g = 0; g < 4; ++g)
            g4[g] = __half2float(scratch[gbase + g * hidden_dim]) + __half2float(ih_t[gbase + g * hidden_dim]);
        float cn, hn;
        flstm_gate(g4[0], g4[1], g4[2], g4[3], __half2float(cell[cbase]), cn, hn);
        cell[cbase] = __float2half(cn);
        hh_next[cbase] = __float2half(hn);
    }
}

// ---- dequantise + transpose [T,N,C] -> [N,T,C] (nn_kernel_cuda.h:416-443) ---------------------
template <bool FP8, int VEC>
__global__ void __launch_bounds__(256)
dequant_transpose_kernel(const uint8_t *__restrict__ in, __half *__restrict__ out,
                         int64_t total_vec, int n_timesteps, int batch_size, int n_channels,
                         float scale) {
    const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total_vec) return;
    const int per_row = n_channels / VEC;
    int64_t tn, t;
    int c, n;
    split_index(idx, total_vec, per_row, tn, c);
    c *= VEC;
    split_index(tn, total_vec, batch_size, t, n);
    const uint8_t *src = in + tn * n_channels + c;
    __half *dst = out + (n * n_timesteps + t) * n_channels + c;
    auto deq = [&](uint8_t b) -> float {
        if constexpr (FP8) return e4m3_decode(b) * scale;
        else return (float)(int8_t)b * scale;
    };
    if constexpr (VEC == 16) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(src));
        const uint8_t *rb = reinterpret_cast<const uint8_t *>(&raw);
        float2 f0[4], f1[4];
        if constexpr (FP8) {
            e4m3x4_decode(raw.x, f0[0], f0[1]);
            e4m3x4_decode(raw.y, f0[2], f0[3]);
            e4m3x4_decode(raw.z, f1[0], f1[1]);
            e4m3x4_decode(raw.w, f1[2], f1[3]);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                f0[k] = make_float2(f0[k].x * scale, f0[k].y * scale);
                f1[k] = make_float2(f1[k].x * scale, f1[k].y * scale);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                f0[k] = make_float2(deq(rb[2 * k]), deq(rb[2 * k + 1]));
                f1[k] = make_float2(deq(rb[8 + 2 * k]), deq(rb[8 + 2 * k + 1]));
            }
        }
        reinterpret_cast<uint4 *>(dst)[0] = pack8(f0);
        reinterpret_cast<uint4 *>(dst)[1] = pack8(f1);
    } else {
        *dst = __float2half(deq(*src));
    }
}

// ---- fp8 weight re-ordering: [N/16, K/16, 2, 16, 8] bytes -> row-major [N, K] -------------------
__global__ void __launch_bounds__(256)
fp8_unshuffle_kernel(uint8_t *__restrict__ dst, const uint8_t *__restrict__ src, int N, int K) {
    // one thread per 8-byte run (fixed n, 8 consecutive k)
    const int64_t idx = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int runs_per_row = K >> 3;
    if (idx >= int64_t(N) * runs_per_row) return;
    const int n = int(idx / runs_per_row), kr = int(idx % runs_per_row);
    const int k0 = kr >> 1, klane = kr & 1, n0 = n >> 4, nl = n & 15;
    const int64_t src_run = ((int64_t(n0) * (K >> 4) + k0) * 2 + klane) * 16 + nl;
    reinterpret_cast<uint2 *>(dst)[idx] = __ldg(reinterpret_cast<const uint2 *>(src) + src_run);
}

inline int grid_for(int64_t total, int block) { return int((total + block - 1) / block); }

}  // namespace
}  // namespace fluke_sm100

using namespace fluke_sm100;

extern "C" int fluke_sm100_rmsnorm(const void *in, const void *residual, const void *weight,
                                   void *out, int n_tokens, int hidden_dim, float alpha, float eps,
                                   void *stream) {
    return launch_rmsnorm<kOutF16>(in, residual, weight, out, nullptr, n_tokens, hidden_dim, alpha,
                                   eps, static_cast<cudaStream_t>(stream));
}

extern "C" int fluke_sm100_rmsnorm_quant_int8(const void *in, const void *weight, void *residual,
                                              void *residual_scale, int n_tokens, int hidden_dim,
                                              float alpha, float eps, void *stream) {
    return launch_rmsnorm<kOutI8>(in, residual, weight, residual, static_cast<float *>(residual_scale),
                                  n_tokens, hidden_dim, alpha, eps, static_cast<cudaStream_t>(stream));
}

extern "C" int fluke_sm100_rmsnorm_quant_fp8(const void *in, const void *weight, void *residual,
                                             void *residual_scale, int n_tokens, int hidden_dim,
                                             float alpha, float eps, void *stream) {
    return launch_rmsnorm<kOutF8>(in, residual, weight, residual, static_cast<float *>(residual_scale),
                                  n_tokens, hidden_dim, alpha, eps, static_cast<cudaStream_t>(stream));
}

static int launch_quant(const void *in, void *out, void *scale, int n_tokens, int hidden_dim,
                        bool fp8, cudaStream_t s) {
    if (n_tokens <= 0) return 0;
    const int vec_ok = (hidden_dim % 8 == 0) &&
                       ((reinterpret_cast<uintptr_t>(in) & 15u) == 0) &&
                       ((reinterpret_cast<uintptr_t>(out) & 7u) == 0);
    if (vec_ok && hidden_dim % 256 == 0 && hidden_dim <= 1024) {
        const __half *x = static_cast<const __half *>(in);
        uint8_t *o = static_cast<uint8_t *>(out);
        float *sc = static_cast<float *>(scale);
        const int grid = (n_tokens + kNormWarps - 1) / kNormWarps, block = kNormWarps * 32;
        switch ((hidden_dim / 256) * 2 + (fp8 ? 1 : 0)) {
            case 2: quant_rows_reg_kernel<1, false><<<grid, block, 0, s>>>(x, o, sc, n_tokens); break;
            case 3: quant_rows_reg_kernel<1, true><<<grid, block, 0, s>>>(x, o, sc, n_tokens); break;
            case 4: quant_rows_reg_kernel<2, false><<<grid, block, 0, s>>>(x, o, sc, n_tokens); break;
            case 5: quant_rows_reg_kernel<2, true><<<grid, block, 0, s>>>(x, o, sc, n_tokens); break;
            case 6: quant_rows_reg_kernel<3, false><<<grid, block, 0, s>>>(x, o, sc, n_tokens); break;
            case 7: quant_rows_reg_kernel<3, true><<<grid, block, 0, s>>>(x, o, sc, n_tokens); break;
            case 8: quant_rows_reg_kernel<4, false><<<grid, block, 0, s>>>(x, o, sc, n_tokens); break;
            default: quant_rows_reg_kernel<4, true><<<grid, block, 0, s>>>(x, o, sc, n_tokens); break;
        }
        return (int)cudaGetLastError();
    }
    const int grid = (n_tokens + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (fp8)
        quant_rows_kernel<true><<<grid, kWarpsPerBlock * 32, 0, s>>>(
            static_cast<const __half *>(in), static_cast<uint8_t *>(out), static_cast<float *>(scale),
            n_tokens, hidden_dim, vec_ok);
    else
        quant_rows_kernel<false><<<grid, kWarpsPerBlock * 32, 0, s>>>(
            static_cast<const __half *>(in), static_cast<uint8_t *>(out), static_cast<float *>(scale),
            n_tokens, hidden_dim, vec_ok);
    return (int)cudaGetLastError();
}

extern "C" int fluke_sm100_quant_int8(const void *in, void *out, void *scale, int n_tokens,
                                      int hidden_dim, void *stream) {
    return launch_quant(in, out, scale, n_tokens, hidden_dim, false, static_cast<cudaStream_t>(stream));
}
extern "C" int fluke_sm100_quant_fp8(const void *in, void *out, void *scale, int n_tokens,
                                     int hidden_dim, void *stream) {
    return launch_quant(in, out, scale, n_tokens, hidden_dim, true, static_cast<cudaStream_t>(stream));
}

extern "C" int fluke_sm100_dequant_transpose(const void *in, void *out, int n_timesteps,
                                             int batch_size, int n_channels, float scale,
                                             int is_fp8, void *stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t rows = int64_t(n_timesteps) * batch_size;
    if (rows <= 0 || n_channels <= 0) return 0;
    const bool vec = (n_channels % 16 == 0) &&
                     (((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0);
    const uint8_t *src = static_cast<const uint8_t *>(in);
    __half *dst = static_cast<__half *>(out);
    if (vec) {
        const int64_t total = rows * (n_channels / 16);
        if (is_fp8) dequant_transpose_kernel<true, 16><<<grid_for(total, 256), 256, 0, s>>>(src, dst, total, n_timesteps, batch_size, n_channels, scale);
        else dequant_transpose_kernel<false, 16><<<grid_for(total, 256), 256, 0, s>>>(src, dst, total, n_timesteps, batch_size, n_channels, scale);
    } else {
        const int64_t total = rows * n_channels;
        if (is_fp8) dequant_transpose_kernel<true, 1><<<grid_for(total, 256), 256, 0, s>>>(src, dst, total, n_timesteps, batch_size, n_channels, scale);
        else dequant_transpose_kernel<false, 1><<<grid_for(total, 256), 256, 0, s>>>(src, dst, total, n_timesteps, batch_size, n_channels, scale);
    }
    return (int)cudaGetLastError();
}

extern "C" int fluke_sm100_rotary_emb(void *x, const void *sin_tab, const void *cos_tab,
                                      int batch_size, int seq_len, int n_heads, int head_dim,
                                      int sincos_width, long long stride_batch,
                                      long long stride_seq, long long stride_head, void *stream) {
    (void)head_dim;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int W = sincos_width;
    if (batch_size <= 0 || seq_len <= 0 || n_heads <= 0 || W <= 0) return 0;
    const bool vec = (W % 8 == 0) && (stride_batch % 8 == 0) && (stride_seq % 8 == 0) &&
                     (stride_head % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) &&
                     (((reinterpret_cast<uintptr_t>(sin_tab) | reinterpret_cast<uintptr_t>(cos_tab)) & 15u) == 0);
    if (vec) {
        const int64_t total = int64_t(batch_size) * seq_len * n_heads * (W / 8);
        const int cpw = W / 8;
        auto log2_of = [](int v) { int l = 0; while ((1 << l) < v) ++l; return (1 << l) == v ? l : -1; };
        const int cl = log2_of(cpw), hl = log2_of(n_heads);
        if (cl >= 0 && hl >= 0 && total < (int64_t(1) << 31)) {
            rotary_vec_kernel<true><<<grid_for(total, 256), 256, 0, s>>>(
                static_cast<__half *>(x), static_cast<const float *>(sin_tab),
                static_cast<const float *>(cos_tab), total, seq_len, n_heads, W, stride_batch,
                stride_seq, stride_head, cl, hl);
        } else {
            rotary_vec_kernel<false><<<grid_for(total, 256), 256, 0, s>>>(
                static_cast<__half *>(x), static_cast<const float *>(sin_tab),
                static_cast<const float *>(cos_tab), total, seq_len, n_heads, W, stride_batch,
                stride_seq, stride_head, 0, 0);
        }
    } else {
        const int64_t total = int64_t(batch_size) * seq_len * n_heads * W;
        rotary_scalar_kernel<<<grid_for(total, 256), 256, 0, s>>>(
            static_cast<__half *>(x), static_cast<const float *>(sin_tab),
            static_cast<const float *>(cos_tab), total, seq_len, n_heads, W, stride_batch,
            stride_seq, stride_head);
    }
    return (int)cudaGetLastError();
}

extern "C" int fluke_sm100_silu_mul(const void *in, void *out, int n_tokens, int hidden_dim,
                                    void *stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (n_tokens <= 0 || hidden_dim <= 0) return 0;
    const bool vec = (hidden_dim % 8 == 0) &&
                     (((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0);
    if (vec) {
        const int64_t total = int64_t(n_tokens) * (hidden_dim / 8);
        silu_mul_kernel<8><<<grid_for(total, 256), 256, 0, s>>>(static_cast<const __half *>(in), static_cast<__half *>(out), total, hidden_dim);
    } else {
        const int64_t total = int64_t(n_tokens) * hidden_dim;
        silu_mul_kernel<1><<<grid_for(total, 256), 256, 0, s>>>(static_cast<const __half *>(in), static_cast<__half *>(out), total, hidden_dim);
    }
    return (int)cudaGetLastError();
}

extern "C" int fluke_sm100_flstm_step(const void *scratch, const void *ih_t, void *cell,
                                      void *hh_next, int batch_size, int hidden_dim, void *stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (batch_size <= 0 || hidden_dim <= 0) return 0;
    const bool vec = (hidden_dim % 8 == 0) &&
                     (((reinterpret_cast<uintptr_t>(scratch) | reinterpret_cast<uintptr_t>(ih_t) |
                        reinterpret_cast<uintptr_t>(cell) | reinterpret_cast<uintptr_t>(hh_next)) & 15u) == 0);
    if (vec) {
        const int64_t total = int64_t(batch_size) * (hidden_dim / 8);
        flstm_step_kernel<8><<<grid_for(total, 256), 256, 0, s>>>(static_cast<const __half *>(scratch), static_cast<const __half *>(ih_t), static_cast<__half *>(cell), static_cast<__half *>(hh_next), total, hidden_dim);
    } else {
        const int64_t total = int64_t(batch_size) * hidden_dim;
        flstm_step_kernel<1><<<grid_for(total, 256), 256, 0, s>>>(static_cast<const __half *>(scratch), static_cast<const __half *>(ih_t), static_cast<__half *>(cell), static_cast<__half *>(hh_next), total, hidden_dim);
    }
    return (int)cudaGetLastError();
}

extern "C" int fluke_sm100_fp8_unshuffle(void *dst_nk, const void *src, int N, int K, void *stream) {
    if (N <= 0 || K <= 0 || N % 16 != 0 || K % 16 != 0) return (int)cudaErrorInvalidValue;
    const int64_t total = int64_t(N) * (K / 8);
    fp8_unshuffle_kernel<<<grid_for(total, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint8_t *>(dst_nk), static_cast<const uint8_t *>(src), N, K);
    return (int)cudaGetLastError();
}
