/*
 * vb_synth.cpp - deterministic synthetic tensors for tests and benchmarks.
 *
 * Stand-in for the real checkpoint (which cannot be fetched offline): BF16
 * matrices ~N(0, sigma) and fp32 vectors ~N(mean, sigma). Integer arithmetic
 * only up to one final fp32 multiply, so every machine produces the same bits:
 *   key  = mix(seed ^ stream * C)
 *   a, b = mix(key + 2i), mix(key + 2i + 1)            (splitmix64 finaliser)
 *   z    = (sum of the 16 bytes of a and b) - 2040     (variance 16 * (256^2-1)/12)
 *   v    = mean + z * (sigma / sqrt(87380))
 * BF16 values are rounded to nearest even from fp32.
 */
#include <stddef.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "../../include/voxtral_b200_ext.h"

static inline uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ULL;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}

static inline int byte_sum(uint64_t v) {
    v = (v & 0x00FF00FF00FF00FFULL) + ((v >> 8) & 0x00FF00FF00FF00FFULL);
    return (int)((v * 0x0001000100010001ULL) >> 48);
}

static inline float unit_normal_times(uint64_t key, uint64_t i, float scale) {
    const int z = byte_sum(mix64(key + 2 * i)) + byte_sum(mix64(key + 2 * i + 1)) - 2040;
    return (float)z * scale;
}

static inline uint16_t f32_to_bf16_rne(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static const float kInvStd = 1.0f / 295.60107f; /* 1/sqrt(87380) */

extern "C" void vb200_synth_bf16(uint16_t *dst, size_t n, uint64_t seed, uint64_t stream, uint64_t first,
                                 float sigma) {
    const uint64_t key = mix64(seed ^ (stream * 0xD6E8FEB86659FD93ULL));
    const float scale = sigma * kInvStd;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; i++)
        dst[i] = f32_to_bf16_rne(unit_normal_times(key, first + (uint64_t)i, scale));
}

extern "C" void vb200_synth_f32(float *dst, size_t n, uint64_t seed, uint64_t stream, uint64_t first,
                                float mean, float sigma) {
    const uint64_t key = mix64(seed ^ (stream * 0xD6E8FEB86659FD93ULL));
    const float scale = sigma * kInvStd;
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; i++)
        dst[i] = mean + unit_normal_times(key, first + (uint64_t)i, scale);
}

/* The reference's noise generator (tts_rng_seed / tts_randn_fill, voxtral_tts_kernels.c:640-669):
 * xorshift64 with shifts 13, 7, 17; uniform = (float)(x >> 11) * 2^-53; Box-Muller, cosine branch
 * only, in single precision with the C library's logf / cosf / sqrtf. For callers of
 * vb200_frame / vb200_utterance_* that do not link the reference's own RNG: they need the 36
 * normals per frame that the reference would draw. state is advanced in place. */
extern "C" void vb200_randn_fill(uint64_t *state, float *out, size_t n) {
    uint64_t x = *state ? *state : 0x12345678ABCDEF01ULL;
    auto uniform = [&x]() {
        x ^= x << 13;
        x ^= x >> 7;
        x ^= x << 17;
        return (float)(x >> 11) * (1.0f / 9007199254740992.0f);
    };
    for (size_t i = 0; i < n; i++) {
        float u1;
        do { u1 = uniform(); } while (u1 < 1e-30f);
        const float u2 = uniform();
        out[i] = sqrtf(-2.0f * logf(u1)) * cosf(6.2831853071795864f * u2);
    }
    *state = x;
}
