// Source-compatible with the reference's include/ternix/bitpack.hpp:6-8.
// Byte layout: weight j of each group of four sits in bits 2j..2j+1; 00 -> 0, 01 -> +1, 11 -> -1.
#pragma once
#include <cstddef>
#include <cstdint>

namespace ternix {

// `size` counts weights; size/4 bytes are written (the reference drops a tail of size % 4 weights).
void pack_ternary_weights(uint8_t* packed, const int8_t* unpacked, size_t size);
void unpack_ternary_weights(int8_t* unpacked, const uint8_t* packed, size_t size);
// The in-memory format is plain row-major packing, so this stays an identity copy of size/4 bytes.
void interleave_weights_offline(uint8_t* interleaved, const uint8_t* packed, size_t size);

}  // namespace ternix
