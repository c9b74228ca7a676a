// Counter-based generator of the synthetic benchmark weights.  Usable from
// host and device code; tensorlogic_b200/synth.py restates it in numpy and the
// tests check that the two produce the same bytes.
//
//   key        = mix64(mix64(seed) ^ tensor_id)
//   r(i)       = mix64(key + i)
//   Q4_0 block b: d = f16_rne(float(2000 + r(3b) % 18001) * 1e-6f * 2^scale_log2)
//                 (U[0.002, 0.02] for scale_log2 = 0; deep random-weight models use
//                 negative exponents so that activations stay inside the f16 range)
//                 qs[0..7] = bytes of r(3b+1), qs[8..15] = bytes of r(3b+2)  (little endian)
//   Q8_0 block b: d as above from r(9b); q[4j..4j+3] = ((u16 * 255) >> 16) - 127 over
//                 the four 16-bit fields of r(9b+1+j), j = 0..7      (U{-127..127})
// where b counts blocks of the FULL (unsharded) tensor in row-major order.
#pragma once
#include <cuda_fp16.h>
#include <cstdint>

__host__ __device__ inline uint64_t tlc_mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__host__ __device__ inline uint64_t tlc_synth_key(uint64_t seed, uint64_t tensor_id) {
    return tlc_mix64(tlc_mix64(seed) ^ tensor_id);
}

__host__ __device__ inline uint16_t tlc_synth_scale_bits(uint64_t r, int scale_log2) {
    float v = (float)(uint32_t)(2000u + (uint32_t)(r % 18001ull));
#ifdef __CUDA_ARCH__
    float d = __fmul_rn(v, 1e-6f);
#else
    volatile float dv = v * 1e-6f;
    float d = dv;
#endif
    d = ldexpf(d, scale_log2);  // exact: a power-of-two factor
    const __half_raw h = __float2half_rn(d);
    return h.x;
}

// Blocks are assembled in 64-bit words and emitted as 16-bit units: a block
// always starts on a 2-byte boundary (18- and 34-byte blocks, 16-byte aligned
// rows), so no store ever touches a neighbouring block's bytes.
__host__ __device__ inline void tlc_synth_put16(uint8_t *dst, uint64_t w, int n_units) {
    uint16_t *d16 = reinterpret_cast<uint16_t *>(dst);
    for (int i = 0; i < n_units; i++) d16[i] = (uint16_t)(w >> (16 * i));
}

__host__ __device__ inline void tlc_synth_q4_0_block(uint64_t key, uint64_t b, int scale_log2, uint8_t *out18) {
    const uint64_t d = tlc_synth_scale_bits(tlc_mix64(key + 3 * b), scale_log2);
    const uint64_t r1 = tlc_mix64(key + 3 * b + 1), r2 = tlc_mix64(key + 3 * b + 2);
    tlc_synth_put16(out18, d | (r1 << 16), 4);                 // d, qs[0..5]
    tlc_synth_put16(out18 + 8, (r1 >> 48) | (r2 << 16), 4);    // qs[6..13]
    tlc_synth_put16(out18 + 16, r2 >> 48, 1);                  // qs[14..15]
}

__host__ __device__ inline void tlc_synth_q8_0_block(uint64_t key, uint64_t b, int scale_log2, uint8_t *out34) {
    const uint64_t d = tlc_synth_scale_bits(tlc_mix64(key + 9 * b), scale_log2);
    tlc_synth_put16(out34, d, 1);
    for (int j = 0; j < 8; j++) {
        const uint64_t r = tlc_mix64(key + 9 * b + 1 + j);
        uint64_t q4 = 0;
        for (int i = 0; i < 4; i++) {
            const uint32_t u = (uint32_t)((r >> (16 * i)) & 0xFFFF);
            q4 |= (uint64_t)(uint8_t)(int8_t)((int)((u * 255u) >> 16) - 127) << (8 * i);
        }
        tlc_synth_put16(out34 + 2 + 4 * j, q4, 2);
    }
}
