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

// How far the screened value may lie from the reference's.  With t = x / scale + zpf in exact arithmetic, the reference
// computes fl(zpf + fl(x / scale)) and the screen fl(x * fl(1 / scale) + zpf) (or the same with one rounding less): each
// is within (|x / scale| + |t|) * 2^-24 of t, and wherever a rounding boundary of the clamp range [0, 255] is in reach
// both magnitudes are below 256, so the two values differ by less than 2 * 512 * 2^-24 = 6.2e-5.  A screened value
// farther than SCREEN_MARGIN (twice that) from every half-integer k + 0.5 therefore rounds to the same byte as the
// reference's (clamping is monotone and its edges 0 and 255 are themselves 0.5 away from the nearest boundary).
constexpr float SCREEN_MARGIN = 1.2e-4f;
constexpr float SCREEN_FAR = 0.5f - SCREEN_MARGIN;   // |v - nearest integer| up to here is safe

// Same result as quant_u8_exact, usually without the division (these kernels are bound by instruction issue, not by
// HBM, and an IEEE division is half of their instructions).  Elements within SCREEN_MARGIN of a rounding boundary, a
// few in ten thousand, take the exact path.
__device__ __forceinline__ uint32_t quant_u8(float x, float scale, float zpf, float inv)
{
    if (inv == 0.f) return quant_u8_exact(x, scale, zpf);
    float v = __fadd_rn(zpf, __fmul_rn(x, inv));
    v = fmaxf(0.f, fminf(255.f, v));
    const float big = __fadd_rn(v, 8388608.f);
    const float r = __fadd_rn(big, -8388608.f);            // nearest integer, |v - r| <= 0.5
    const float d = fabsf(__fsub_rn(v, r));
    if (d > SCREEN_FAR) return quant_u8_exact(x, scale, zpf);
    return __float_as_uint(big) & 0xFFu;
}

// The rarely taken branch of quant4_u8 (a warp enters it when any of its 128 elements is within SCREEN_MARGIN of a
// rounding boundary: two or three warps in a hundred): only the elements that are close get the reference's sequence
// with its division - as a rule one of the four - the others keep the screened byte.  Out of line so that it costs the
// callers' hot loops neither registers nor instruction-cache room.  inv == 0 (no screening possible): all four exact.
static __device__ __noinline__ uint32_t quant4_u8_careful(float4 x, float scale, float zpf, float inv)
{
    uint32_t out = 0;
    const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float v = fmaxf(0.f, fminf(255.f, fmaf(xs[k], inv, zpf)));
        const float b = __fadd_rn(v, 8388608.f);
        const float d = fabsf(__fsub_rn(v, __fadd_rn(b, -8388608.f)));
        uint32_t byte = __float_as_uint(b) & 0xFFu;
        if (inv == 0.f || d > SCREEN_FAR) byte = quant_u8_exact(xs[k], scale, zpf);
        out |= byte << (8 * k);
    }
    return out;
}

// Four elements at once, packed little-endian into one word.  The screening value may come from a fused multiply-add
// (one rounding less than separate operations); the bytes are taken from the low mantissa bytes of v + 2^23 with three
// byte permutes.
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
        const bool near = fmaxf(fmaxf(fabsf(d0), fabsf(d1)), fmaxf(fabsf(d2), fabsf(d3))) > SCREEN_FAR;
        if (!near) {
            const uint32_t lo = __byte_perm(__float_as_uint(b0), __float_as_uint(b1), 0x0040);  // bytes b0[0], b1[0]
            const uint32_t hi = __byte_perm(__float_as_uint(b2), __float_as_uint(b3), 0x0040);
            return __byte_perm(lo, hi, 0x5410);
        }
    }
    return quant4_u8_careful(x, scale, zpf, inv);
}

}  // namespace ltq
