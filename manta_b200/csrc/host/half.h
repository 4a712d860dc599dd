// f32 -> f16 conversion shared by the host-side components.
#pragma once

#include <cstdint>
#include <cstring>

namespace mb200_host {

// f32 -> f16 bits, round to nearest even (the kernels take IEEE half bits).
inline uint16_t half_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u, absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x0200u : 0));
    if (absx >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);
    if (absx < 0x33000001u) return (uint16_t)sign;
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x007fffffu) | 0x00800000u, shift, base;
    if (e < -14) { shift = (uint32_t)(13 + (-14 - e)); base = 0; }
    else { shift = 13; base = ((uint32_t)(e + 15) << 10) - 0x0400u; }
    uint32_t q = m >> shift, rem = m & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    return (uint16_t)(sign | (base + q));
}

}  // namespace mb200_host
