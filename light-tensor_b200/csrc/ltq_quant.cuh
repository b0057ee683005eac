// Device-side arithmetic of Quantize(float -> uint8), l-ten/utils.cpp:243-254, shared by the quantise kernels and the
// fused MLP kernel: the reference's exact sequence, and a division-free screened form that gives the same bytes.
#pragma once
#include <stdint.h>

namespace ltq {

// round(v), half away from zero, for v in [0, 255] without the conversion unit: adding 2^23 rounds to the nearest integer
// with ties to even; the only difference from half-away is a tie that went DOWN (v = r + 0.5 with r even), which is put
// right by one comparison.  The integer is then read from the low mantissa bits.
__device__ __forceinline__ uint32_t round_u8(float v)
{
    float r = __fadd_rn(__fadd_rn(v, 8388608.f), -8388608.f);
    if (__fsub_rn(v, r) == 0.5f) r = __fadd_rn(r, 1.f);
    return __float_as_uint(__fadd_rn(r, 8388608.f)) & 0xFFu;
}

// The reference's arithmetic to the letter (l-ten/utils.cpp:249-251): IEEE division, add, clamp, round.
__device__ __forceinline__ uint32_t quant_u8_exact(float x, float scale, float zpf)
{
    float v = __fadd_rn(zpf, __fdiv_rn(x, scale));
    v = fmaxf(0.f, fminf(255.f, v));
    return round_u8(v);
}

// Multiplier for the screening step below, or 0 when the scale is too extreme for the screening bound to hold.
__device__ __forceinline__ float quant_screen_inv(float scale)
{
    return (scale > 1e-30f && scale < 1e30f) ? __fdiv_rn(1.f, scale) : 0.f;
}

// Same result as quant_u8_exact, usually without the division (these kernels are bound by instruction issue, not by
// HBM, and an IEEE division is half of their instructions).  x * (1/scale) differs from x / scale by at most 2^-22
// relative; inside the clamp range that is less than 1.3e-4 absolute on v, so whenever the screened v lies farther than
// 4e-4 from every half-integer k + 0.5 both round to the same byte (clamping is monotone and its edges 0 and 255 are
// themselves 0.5 away from the nearest rounding boundary).  Elements closer than that, a few in ten thousand, take the
// exact path.
__device__ __forceinline__ uint32_t quant_u8(float x, float scale, float zpf, float inv)
{
    if (inv == 0.f) return quant_u8_exact(x, scale, zpf);
    float v = __fadd_rn(zpf, __fmul_rn(x, inv));
    v = fmaxf(0.f, fminf(255.f, v));
    const float big = __fadd_rn(v, 8388608.f);
    const float r = __fadd_rn(big, -8388608.f);            // nearest integer, |v - r| <= 0.5
    const float d = fabsf(__fsub_rn(v, r));
    if (__fsub_rn(0.5f, d) < 4e-4f) return quant_u8_exact(x, scale, zpf);
    return __float_as_uint(big) & 0xFFu;
}

// The reference's sequence for four elements.  Rarely taken (a few warps in a hundred): kept out of line so that its four
// divisions cost the callers' hot loops neither registers nor instruction-cache room.
static __device__ __noinline__ uint32_t quant4_u8_exact(float4 x, float scale, float zpf)
{
    return quant_u8_exact(x.x, scale, zpf) | (quant_u8_exact(x.y, scale, zpf) << 8) |
           (quant_u8_exact(x.z, scale, zpf) << 16) | (quant_u8_exact(x.w, scale, zpf) << 24);
}

// Four elements at once, packed little-endian into one word.  The screening value may come from a fused multiply-add
// (it only has to be within 1.3e-4 of the reference's v, and an FMA is closer than separate roundings); the bytes are
// taken from the low mantissa bytes of v + 2^23 with three byte permutes.  If any of the four lies within 4e-4 of a
// rounding boundary, all four are redone with the reference's exact sequence.
__device__ __forceinline__ uint32_t quant4_u8(float4 x, float scale, float zpf, float inv)
{
    if (inv != 0.f) {
        const float v0 = fmaxf(0.f, fminf(255.f, fmaf(x.x, inv, zpf))), v1 = fmaxf(0.f, fminf(255.f, fmaf(x.y, inv, zpf)));
        const float v2 = fmaxf(0.f, fminf(255.f, fmaf(x.z, inv, zpf))), v3 = fmaxf(0.f, fminf(255.f, fmaf(x.w, inv, zpf)));
        const float b0 = __fadd_rn(v0, 8388608.f), b1 = __fadd_rn(v1, 8388608.f);
        const float b2 = __fadd_rn(v2, 8388608.f), b3 = __fadd_rn(v3, 8388608.f);
        const float d0 = __fsub_rn(v0, __fadd_rn(b0, -8388608.f)), d1 = __fsub_rn(v1, __fadd_rn(b1, -8388608.f));
        const float d2 = __fsub_rn(v2, __fadd_rn(b2, -8388608.f)), d3 = __fsub_rn(v3, __fadd_rn(b3, -8388608.f));
        // one comparison on the largest distance (four short-circuited comparisons are four branches)
        const bool near = fmaxf(fmaxf(fabsf(d0), fabsf(d1)), fmaxf(fabsf(d2), fabsf(d3))) > 0.4996f;
        if (!near) {
            const uint32_t lo = __byte_perm(__float_as_uint(b0), __float_as_uint(b1), 0x0040);  // bytes b0[0], b1[0]
            const uint32_t hi = __byte_perm(__float_as_uint(b2), __float_as_uint(b3), 0x0040);
            return __byte_perm(lo, hi, 0x5410);
        }
    }
    return quant4_u8_exact(x, scale, zpf);
}

}  // namespace ltq
