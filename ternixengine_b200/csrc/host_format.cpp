// Host side of the packed ternary weight format, column sharding of packed matrices and the
// seeded synthetic-input generator.  C++20, no CUDA.  Declared in include/ternix_b200.h.
#include "ternix_b200.h"

#include <algorithm>
#include <bit>
#include <cstring>
#include <thread>
#include <vector>

namespace {

// weight value -> 2-bit code: +1 -> 01, -1 -> 11, everything else -> 00
constexpr uint8_t code_of(int8_t v) { return v == 1 ? 1u : v == -1 ? 3u : 0u; }

// splitmix64 finaliser applied to a counter: random access, no state
constexpr uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
constexpr uint64_t stream_key(uint64_t seed) { return mix64(seed ^ 0xA5A5A5A55A5A5A5Aull); }

// P(-1) = P(+1) = 0.3, P(0) = 0.4, decided by the top 32 bits of the hash
constexpr uint32_t kCutNeg = 1288490189u;   // floor(0.3 * 2^32)
constexpr uint32_t kCutPos = 2576980378u;   // floor(0.6 * 2^32)
constexpr int8_t ternary_of(uint64_t h) {
    const uint32_t u = static_cast<uint32_t>(h >> 32);
    return u < kCutNeg ? int8_t(-1) : u < kCutPos ? int8_t(1) : int8_t(0);
}

template <class F>
void parallel_ranges(size_t n, size_t grain, F&& body) {
    unsigned hw = std::thread::hardware_concurrency();
    if (hw == 0) hw = 1;
    const size_t parts = std::min<size_t>(hw, std::max<size_t>(1, n / grain));
    if (parts <= 1) { body(size_t(0), n); return; }
    std::vector<std::thread> pool;
    const size_t step = (n + parts - 1) / parts;
    for (size_t b = 0; b < n; b += step) pool.emplace_back([=, &body] { body(b, std::min(n, b + step)); });
    for (auto& t : pool) t.join();
}

}  // namespace

extern "C" {

void ternix_b200_pack_ternary(uint8_t* packed, const int8_t* unpacked, size_t size) {
    const size_t n = size / 4;
    parallel_ranges(n, size_t(1) << 20, [=](size_t b, size_t e) {
        for (size_t g = b; g < e; ++g) {
            const int8_t* v = unpacked + 4 * g;
            packed[g] = static_cast<uint8_t>(code_of(v[0]) | code_of(v[1]) << 2 | code_of(v[2]) << 4 | code_of(v[3]) << 6);
        }
    });
}

void ternix_b200_unpack_ternary(int8_t* unpacked, const uint8_t* packed, size_t size) {
    const size_t n = size / 4;
    parallel_ranges(n, size_t(1) << 20, [=](size_t b, size_t e) {
        for (size_t g = b; g < e; ++g) {
            const unsigned byte = packed[g];
            for (int f = 0; f < 4; ++f) {
                const unsigned c = (byte >> (2 * f)) & 3u;
                unpacked[4 * g + f] = c == 1u ? int8_t(1) : c == 3u ? int8_t(-1) : int8_t(0);
            }
        }
    });
}

void ternix_b200_interleave_offline(uint8_t* interleaved, const uint8_t* packed, size_t size) {
    if (size / 4) std::memmove(interleaved, packed, size / 4);
}

long long ternix_b200_find_non_ternary(const int8_t* unpacked, size_t size) {
    for (size_t i = 0; i < size; ++i)
        if (unpacked[i] < -1 || unpacked[i] > 1) return static_cast<long long>(i);
    return -1;
}

int ternix_b200_slice_columns(uint8_t* dst, const uint8_t* packed, size_t K, size_t N, size_t n0, size_t n_cols) {
    if ((N % 4) || (n0 % 4) || (n_cols % 4) || n0 + n_cols > N) return TERNIX_B200_ERR_INVALID_SHAPE;
    if (K && n_cols && (!dst || !packed)) return TERNIX_B200_ERR_INVALID_ARG;
    const size_t src_pitch = N / 4, dst_pitch = n_cols / 4, off = n0 / 4;
    for (size_t k = 0; k < K; ++k) std::memcpy(dst + k * dst_pitch, packed + k * src_pitch + off, dst_pitch);
    return TERNIX_B200_OK;
}

void ternix_b200_synth_activations(int8_t* A, size_t count, uint64_t seed, int mode) {
    const uint64_t key = stream_key(seed);
    parallel_ranges(count, size_t(1) << 20, [=](size_t b, size_t e) {
        for (size_t i = b; i < e; ++i) {
            const uint64_t h = mix64(key + i);
            A[i] = mode == 1 ? static_cast<int8_t>(static_cast<int>(h % 255u) - 127)
                             : std::bit_cast<int8_t>(static_cast<uint8_t>(h & 0xFFu));
        }
    });
}

void ternix_b200_synth_weights(int8_t* W, size_t K, size_t N, uint64_t seed) {
    const uint64_t key = stream_key(seed ^ 0x57454947ull);
    parallel_ranges(K * N, size_t(1) << 20, [=](size_t b, size_t e) {
        for (size_t i = b; i < e; ++i) W[i] = ternary_of(mix64(key + i));
    });
}

void ternix_b200_synth_packed_weights(uint8_t* W_packed, size_t K, size_t N, uint64_t seed) {
    const uint64_t key = stream_key(seed ^ 0x57454947ull);
    const size_t n = K * N / 4;
    parallel_ranges(n, size_t(1) << 18, [=](size_t b, size_t e) {
        for (size_t g = b; g < e; ++g) {
            unsigned byte = 0;
            for (int f = 0; f < 4; ++f) byte |= code_of(ternary_of(mix64(key + 4 * g + f))) << (2 * f);
            W_packed[g] = static_cast<uint8_t>(byte);
        }
    });
}

}  // extern "C"
