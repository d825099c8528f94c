/*
 * TEST INFRASTRUCTURE — CPU restatement of AdaCode's float11 bit-plane codec.
 *
 * This file is the parity oracle and the timed CPU baseline.  It is never
 * linked into, imported by, or called from the shipped CUDA path; only the
 * tests, the smoke check and the benchmark's cpu_baseline / reference arm may
 * load it.
 *
 * Parity status: PINNED.  The Python loader beside this file is checked against
 * byte vectors produced by the reference's own pack code (pure-torch
 * compress_open_tiled_rows + seal_open_tiled_rows and the Triton kernels under
 * the interpreter); see tests/golden/.
 *
 * Format restated here (all citations are paths inside the reference project):
 *   window        left = right - 2**nbits + 1, coded range (left, right]
 *                 compress_bitmap_merge.py:648-650
 *   escape rule   exp <= left or exp > right        compress_bitmap_merge.py:196-197
 *   sign/mantissa ((x >> 8) & 0x80) | (x & 0x7F)    compress_bitmap_merge.py:280-283
 *   code          exp - left if 0 <= exp-left < 2**nbits else 0
 *                 compress_bitmap_merge.py:287-293 (and :336-342, :371-377, :406-412)
 *   bit packing   8 consecutive codes form one big-endian nbits-byte word with
 *                 element 0 in the most significant bits
 *                 compress_bitmap_merge.py:297-315, compress_tiled_kv.py:448-466
 *   escapes       raw exponents of escaped elements in flat [b][h][s][d] order
 *                 compress_bitmap_merge.py:249
 *   tile base     inclusive running escape count at the end of each (b,h) tile
 *                 compress_bitmap_merge.py:250, compress_tiled_kv.py:568-569
 *   histogram     256 bins over the exponent of every element
 *                 compress_bitmap_merge.py:205-208, compress_tiled_kv.py:503-504
 *   decode        compress_tiled_kv.py:33-93
 *   adjuster      float_cache_utils.py:373-398
 *   calibration   best_bit_analysis_kv_cache.py:28-59
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

static inline int is_escape(int e, int left, int right) { return e <= left || e > right; }

/*
 * Pack one segment: n_tiles tiles of tile_elems bf16 values each, already in
 * flat [b][h][s][d] order (x holds the raw 16-bit patterns).
 *
 * Outputs: sign_mant[n], codes[n*nbits/8], escapes (capacity n), tile_base[n_tiles]
 * (inclusive cumulative), hist[256] (added to, may be NULL).  Returns the number
 * of escapes, or -1 for bad arguments.
 */
int64_t oracle_pack_segment(const uint16_t *x, int64_t n_tiles, int64_t tile_elems, int right, int nbits,
                            uint8_t *sign_mant, uint8_t *codes, uint8_t *escapes, int32_t *tile_base,
                            int64_t *hist) {
    if (nbits < 1 || nbits > 4 || tile_elems % 8 != 0 || n_tiles < 0) return -1;
    const int left = right - (1 << nbits) + 1;
    int64_t *counts = (int64_t *)calloc((size_t)(n_tiles > 0 ? n_tiles : 1), sizeof(int64_t));
    if (!counts) return -1;

    /* pass 1: escape count per tile (compress_bitmap_merge.py:196-203) */
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < n_tiles; ++t) {
        const uint16_t *p = x + t * tile_elems;
        int64_t c = 0;
        for (int64_t i = 0; i < tile_elems; ++i) c += is_escape((p[i] >> 7) & 0xFF, left, right);
        counts[t] = c;
    }
    /* inclusive prefix (compress_bitmap_merge.py:250; compress_tiled_kv.py:568-569) */
    int64_t run = 0;
    for (int64_t t = 0; t < n_tiles; ++t) {
        run += counts[t];
        tile_base[t] = (int32_t)run;
    }

    /* pass 2: planes + escape bytes */
#pragma omp parallel
    {
        int64_t local_hist[256];
        memset(local_hist, 0, sizeof(local_hist));
#pragma omp for schedule(static)
        for (int64_t t = 0; t < n_tiles; ++t) {
            const uint16_t *p = x + t * tile_elems;
            uint8_t *sm = sign_mant + t * tile_elems;
            uint8_t *cd = codes + (t * tile_elems / 8) * nbits;
            uint8_t *esc = escapes + (tile_base[t] - counts[t]);
            for (int64_t g = 0; g < tile_elems / 8; ++g) {
                uint32_t word = 0;
                for (int k = 0; k < 8; ++k) {
                    const uint32_t v = p[g * 8 + k];
                    const int e = (v >> 7) & 0xFF;
                    sm[g * 8 + k] = (uint8_t)(((v >> 8) & 0x80) | (v & 0x7F));
                    local_hist[e]++;
                    uint32_t code = 0;
                    if (is_escape(e, left, right)) *esc++ = (uint8_t)e;
                    else code = (uint32_t)(e - left);
                    word |= code << ((7 - k) * nbits);
                }
                for (int b = 0; b < nbits; ++b) cd[g * nbits + b] = (uint8_t)(word >> (8 * (nbits - 1 - b)));
            }
        }
        if (hist) {
#pragma omp critical
            for (int i = 0; i < 256; ++i) hist[i] += local_hist[i];
        }
    }
    free(counts);
    return run;
}

/*
 * Unpack one segment (compress_tiled_kv.py:33-93): tile t's escapes start at
 * tile_base[t-1] (0 for the first tile) and are consumed in flat order by the
 * elements whose code is 0.  Returns 0, or -1 for bad arguments, or -2 when a
 * tile asks for an escape beyond n_escapes.
 */
int oracle_unpack_segment(const uint8_t *sign_mant, const uint8_t *codes, const uint8_t *escapes,
                          int64_t n_escapes, const int32_t *tile_base, int64_t n_tiles, int64_t tile_elems,
                          int left, int nbits, uint16_t *out) {
    if (nbits < 1 || nbits > 4 || tile_elems % 8 != 0) return -1;
    int status = 0;
    const uint32_t mask = (1u << nbits) - 1u;
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < n_tiles; ++t) {
        const uint8_t *sm = sign_mant + t * tile_elems;
        const uint8_t *cd = codes + (t * tile_elems / 8) * nbits;
        int64_t rank = t > 0 ? tile_base[t - 1] : 0;
        uint16_t *o = out + t * tile_elems;
        for (int64_t g = 0; g < tile_elems / 8; ++g) {
            uint32_t word = 0;
            for (int b = 0; b < nbits; ++b) word = (word << 8) | cd[g * nbits + b];
            for (int k = 0; k < 8; ++k) {
                const uint32_t code = (word >> ((7 - k) * nbits)) & mask;
                uint32_t e;
                if (code == 0) {
                    if (rank >= n_escapes) {
                        status = -2;
                        e = 0;
                    } else {
                        e = escapes[rank];
                    }
                    rank++;
                } else {
                    e = code + (uint32_t)left;
                }
                const uint32_t s = sm[g * 8 + k];
                o[g * 8 + k] = (uint16_t)(((s & 0x80u) << 8) | (s & 0x7Fu) | ((e & 0xFFu) << 7));
            }
        }
    }
    return status;
}

/* 256-bin exponent histogram of n raw bf16 patterns, added into hist
 * (float_cache_utils.py:883-891). */
void oracle_hist(const uint16_t *x, int64_t n, int64_t *hist) {
#pragma omp parallel
    {
        int64_t local_hist[256];
        memset(local_hist, 0, sizeof(local_hist));
#pragma omp for schedule(static)
        for (int64_t i = 0; i < n; ++i) local_hist[(x[i] >> 7) & 0xFF]++;
#pragma omp critical
        for (int i = 0; i < 256; ++i) hist[i] += local_hist[i];
    }
}

/* Order of bins by count, descending, equal counts keeping ascending bin order
 * (Python's stable sorted(..., reverse=True), float_cache_utils.py:378). */
static void stable_order_desc(const int64_t *hist, int *order) {
    for (int i = 0; i < 256; ++i) order[i] = i;
    for (int i = 1; i < 256; ++i) { /* insertion sort is stable */
        const int idx = order[i];
        int j = i - 1;
        while (j >= 0 && hist[order[j]] < hist[idx]) {
            order[j + 1] = order[j];
            --j;
        }
        order[j + 1] = idx;
    }
}

/*
 * Run-time adjuster (float_cache_utils.py:373-398): code lengths 2,3,4 with
 * 2**n - 1 coded bins, cost total*n + outliers*8, strict improvement only.
 * Returns 0 and fills right/nbits, or -1 where the reference raises IndexError
 * (no candidate beats 8 bits per exponent).
 */
int oracle_choose_params(const int64_t *hist, int *right, int *nbits) {
    int order[256];
    stable_order_desc(hist, order);
    int64_t total = 0;
    for (int i = 0; i < 256; ++i) total += hist[i];
    int64_t best = total * 8;
    int best_n = 0, best_right = -1;
    for (int n = 2; n <= 4; ++n) {
        const int space = (1 << n) - 1;
        int64_t covered = 0;
        int mx = -1;
        for (int k = 0; k < space; ++k) {
            covered += hist[order[k]];
            if (order[k] > mx) mx = order[k];
        }
        const int64_t cost = total * n + (total - covered) * 8;
        if (cost < best) {
            best = cost;
            best_n = n;
            best_right = mx;
        }
    }
    if (best_n == 0) return -1;
    *right = best_right;
    *nbits = best_n;
    return 0;
}

/*
 * Offline calibration rule (best_bit_analysis_kv_cache.py:28-59): code lengths
 * 1..8 with 2**n coded bins.  Same return convention as above.
 */
int oracle_calibrate_coo(const int64_t *hist, int *right, int *nbits) {
    int order[256];
    stable_order_desc(hist, order);
    int64_t total = 0;
    for (int i = 0; i < 256; ++i) total += hist[i];
    int64_t best = total * 8;
    int best_n = 0, best_right = -1;
    for (int n = 1; n <= 8; ++n) {
        const int space = 1 << n;
        int64_t covered = 0;
        int mx = -1;
        for (int k = 0; k < space && k < 256; ++k) {
            covered += hist[order[k]];
            if (order[k] > mx) mx = order[k];
        }
        const int64_t cost = total * n + (total - covered) * 8;
        if (cost < best) {
            best = cost;
            best_n = n;
            best_right = mx;
        }
    }
    if (best_n == 0) return -1;
    *right = best_right;
    *nbits = best_n;
    return 0;
}
