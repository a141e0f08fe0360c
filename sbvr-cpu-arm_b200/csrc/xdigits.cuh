// Activations -> the B operand of the FP4 tensor-core GEMV: block fixed point, radix-4 E2M1 digits.
//
// One 256-k block of one activation row becomes 1024 bytes laid out [kw (8)][digit (8)][16 B]: the 16 bytes of
// (kw, digit) hold the 32 elements k = 32 kw + 4 i + j as 4-bit E2M1 codes, word j, nibble i -- the K permutation
// in which the weight expansion `w & 0x1111.., w & 0x2222.., w & 0x4444.., (w >> 1) & 0x4444..` leaves the
// plane bits.  q = round(x / step) is 16-bit two's complement with a power-of-two step per group; digits 0..6 are
// q's bit pairs {0,1,2,3}, digit 7 is signed {0,1,-2,-1}; each is pre-multiplied by 2, 1, 0.5, 0.5 for j = 0..3 to
// undo the weights 0.5, 1, 2, 2 the expansion gives the plane bits.  All of these are exact E2M1 values.
#pragma once

#include "common.cuh"

namespace sbvr {

// One warp turns the 256 fp16 activations in the first 512 bytes of `area` (shared memory, 1024 bytes, 16-byte
// aligned) into the 1024 digit bytes, in place.  NSUB = 256 / G groups share the block; their steps go to
// step_out[0 .. NSUB-1] (written by one lane each).  Non-finite activations poison their group (step = NaN).
template <int NSUB>
__device__ __forceinline__ void xdigits_block(unsigned char* area, float* step_out, int lane) {
    // lane (kw, j) owns the eight elements k = 32 kw + j + 4 e, which are exactly one 32-bit word of every digit plane
    const int kw = lane >> 2, j = lane & 3;
    // E2M1 codes of digit value t = 0..3 as bytes, scaled by 2, 1, 0.5, 0.5 for j = 0..3; the low digits
    // take t as {0,1,2,3}, the top digit as {0,1,-2,-1}
    const uint32_t pool_lo = (j == 0) ? 0x07060400u : (j == 1) ? 0x05040200u : 0x03020100u;
    const uint32_t pool_hi = (j == 0) ? 0x0C0E0400u : (j == 1) ? 0x0A0C0200u : 0x090A0100u;
    // Digit words are stored rotated by kw (word i of this lane is digit (i + kw) & 7) so that the eight
    // kw of a warp hit different banks; the rotation is applied to the digits themselves, which keeps
    // every register index static.  `top` marks the nibble that holds digit 7 after the rotation.
    const uint32_t rot = 4u * (uint32_t)kw;
    const uint32_t top = 4u << (4u * (uint32_t)(7 - kw));
    const __half* xp = reinterpret_cast<const __half*>(area) + 32 * kw + j;
    float v[8];
    float a = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        v[e] = __half2float(xp[4 * e]);
        float av = fabsf(v[e]);
        if (!(av == av)) av = __int_as_float(0x7f800000);     // NaN counts as infinity
        a = fmaxf(a, av);
    }
    __syncwarp();                      // all lanes hold their elements: the area may be overwritten
#pragma unroll
    for (int o = (NSUB == 2 ? 8 : 16); o; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    float step = 0.0f, inv = 0.0f;
    bool poison = false;
    if (a >= __int_as_float(0x7f800000)) {                    // non-finite activations poison the group
        step = __int_as_float(0x7fc00000);
        poison = true;
    } else if (a > 0.0f) {
        const int ex = (int)((__float_as_uint(a) >> 23) & 0xFF) - 127;   // a = 1.f * 2^ex, ex in [-24, 15]
        step = __uint_as_float((uint32_t)(ex - 14 + 127) << 23);
        inv = __uint_as_float((uint32_t)(14 - ex + 127) << 23);
    }
    if (NSUB == 1) {
        if (lane == 0) step_out[0] = step;
    } else {
        if ((lane & 15) == 0) step_out[lane >> 4] = step;
    }
    // per element: 16-bit two's complement -> its 8 radix-4 digits, one per nibble -> rotate -> codes
    uint32_t c_lo[8], c_hi[8];         // bytes i = 0..3 / 4..7: code of rotated digit i
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const uint32_t q = poison ? 1u : (uint32_t)__float2int_rn(v[e] * inv);     // |q| < 2^15
        uint32_t sp = __byte_perm(q, 0u, 0x4140);                 // bytes [q0, 0, q1, 0]
        sp = (sp | (sp << 4)) & 0x0F0F0F0Fu;
        sp = (sp | (sp << 2)) & 0x33333333u;                      // nibble d = digit d
        sp = __funnelshift_r(sp, sp, rot) | top;                  // nibble i = digit (i + kw) & 7; top digit + 4
        c_lo[e] = __byte_perm(pool_lo, pool_hi, sp);
        c_hi[e] = __byte_perm(pool_lo, pool_hi, sp >> 16);
    }
    // element pairs share a byte (low nibble = even element), then a 4 x 4 byte transpose per half
    uint32_t* dstw = reinterpret_cast<uint32_t*>(area) + kw * 32 + j;
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
        uint32_t R[4];
#pragma unroll
        for (int pr = 0; pr < 4; ++pr)
            R[pr] = hf ? (c_hi[2 * pr] | (c_hi[2 * pr + 1] << 4)) : (c_lo[2 * pr] | (c_lo[2 * pr + 1] << 4));
        const uint32_t t0 = __byte_perm(R[0], R[1], 0x5140), t1 = __byte_perm(R[2], R[3], 0x5140);
        const uint32_t t2 = __byte_perm(R[0], R[1], 0x7362), t3 = __byte_perm(R[2], R[3], 0x7362);
        const uint32_t T[4] = {__byte_perm(t0, t1, 0x5410), __byte_perm(t0, t1, 0x7632),
                               __byte_perm(t2, t3, 0x5410), __byte_perm(t2, t3, 0x7632)};
#pragma unroll
        for (int i = 0; i < 4; ++i) dstw[(((hf * 4 + i) + kw) & 7) * 4] = T[i];   // [kw][digit][16 B], word j
    }
}

}  // namespace sbvr
