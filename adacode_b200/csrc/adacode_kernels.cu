// float11 KV-cache codec for B200 (sm_100a): pack, unpack, exponent histogram and the
// code-length adjuster, behind the C ABI declared in include/adacode.h.
//
// Work decomposition shared by pack and unpack
//   tile   = seq_tile tokens x D dims of one (batch, kv head)           (contiguous planes)
//   chunk  = CH consecutive elements of a tile (CH = 16, or 8 when D % 16 != 0);
//            one thread moves one chunk with 128-bit (CH=16) loads/stores
//   slab   = 256 threads x 4 chunks, walked in (warp, k, lane) order so that every
//            warp-level access is a contiguous run and the escape rank of an element is
//            a warp scan plus an 8-entry cross-warp prefix
// Both kernels are bandwidth work: no tensor cores, no reshaping into GEMMs.
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "adacode.h"

namespace {

thread_local char g_last_cuda_error[256] = "";

int cuda_fail(cudaError_t e) {
    strncpy(g_last_cuda_error, cudaGetErrorString(e), sizeof(g_last_cuda_error) - 1);
    return ADACODE_ERR_CUDA;
}

#define ADACODE_CUDA_TRY(expr)                        \
    do {                                              \
        cudaError_t e__ = (expr);                     \
        if (e__ != cudaSuccess) return cuda_fail(e__); \
    } while (0)

int g_sm_count = 0;
int sm_count() {
    if (g_sm_count == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        g_sm_count = n;
    }
    return g_sm_count;
}

#include "adacode_device.cuh"

// ---------------------------------------------------------------------------------------
// pack
// ---------------------------------------------------------------------------------------

struct PackArgs {
    const uint16_t *src;
    int64_t sb, sh, ss;      // element strides of src
    int H, BH, seq_tile, D;
    int left;
    int64_t n_tiles;
    int tile_elems;          // seq_tile * D
    int chunks_per_tile;     // tile_elems / CH
    int tile_code_bytes;     // tile_elems * N / 8
    uint8_t *sign_mant;
    uint8_t *codes;
    uint8_t *esc_scratch;    // n_tiles * tile_elems bytes, tile t owns [t*tile_elems, ...)
    int32_t *tile_counts;    // n_tiles
    unsigned int *done;      // zero on entry, zero on exit
    int32_t *tile_base;      // n_tiles, out
    int64_t *seg_off;        // n_blocks + 1, out
    int n_blocks;
    int32_t *hist;           // nullable
};

template <int N, int CH, bool HIST>
__global__ void __launch_bounds__(kThreads) k_pack(const PackArgs a) {
    constexpr int W = CH / 8;              // uint4 loads (and code groups) per chunk
    constexpr int CB = CH * N / 8;         // code bytes per chunk
    __shared__ __align__(16) uint8_t s_codes[kSlabChunks * CB];
    __shared__ int s_warp_tot[kWarps];
    __shared__ int s_hist[HIST ? 256 : 1];
    __shared__ int s_is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t cnt[1 << N];
#pragma unroll
    for (int v = 0; v < (1 << N); ++v) cnt[v] = 0;
    if (HIST) {
        s_hist[tid] = 0;
        __syncthreads();
    }
    const bool rows_contig = (a.ss == a.D);
    const int n_slabs = (a.chunks_per_tile + kSlabChunks - 1) / kSlabChunks;

    for (int64_t tile = blockIdx.x; tile < a.n_tiles; tile += gridDim.x) {
        const int64_t blk = tile / a.BH;
        const int bh = (int)(tile - blk * a.BH);
        const int b = bh / a.H, h = bh - b * a.H;
        const uint16_t *tsrc = a.src + (int64_t)b * a.sb + (int64_t)h * a.sh + blk * a.seq_tile * a.ss;
        uint8_t *tsm = a.sign_mant + tile * a.tile_elems;
        uint8_t *tcodes = a.codes + tile * a.tile_code_bytes;
        uint8_t *tesc = a.esc_scratch + tile * a.tile_elems;
        int running = 0;

        for (int slab = 0; slab < n_slabs; ++slab) {
            uint4 w[kCPT][W];
            const uint16_t *cptr[kCPT];
            int cidx[kCPT];
#pragma unroll
            for (int k = 0; k < kCPT; ++k) {
                const int c = slab * kSlabChunks + warp * (kCPT * 32) + k * 32 + lane;
                cidx[k] = c;
                const bool valid = c < a.chunks_per_tile;
                const int e0 = c * CH;
                int64_t off;
                if (rows_contig) {
                    off = e0;
                } else {
                    const int row = e0 / a.D;
                    off = (int64_t)row * a.ss + (e0 - row * a.D);
                }
                cptr[k] = tsrc + off;
#pragma unroll
                for (int q = 0; q < W; ++q)
                    w[k][q] = valid ? __ldcs(reinterpret_cast<const uint4 *>(cptr[k]) + q) : make_uint4(0, 0, 0, 0);
            }

            int zc[kCPT];
            uint32_t zm[kCPT][W];
#pragma unroll
            for (int k = 0; k < kCPT; ++k) {
                const bool valid = cidx[k] < a.chunks_per_tile;
                uint32_t g[W];
                zc[k] = 0;
#pragma unroll
                for (int q = 0; q < W; ++q) {
                    const uint32_t ww[4] = {w[k][q].x, w[k][q].y, w[k][q].z, w[k][q].w};
                    g[q] = encode_group<N>(ww, a.left);
                    zm[k][q] = valid ? zero_slots<N>(g[q]) : 0u;
                    zc[k] += __popc(zm[k][q]);
                    if (HIST && valid) count_codes<N>(g[q], cnt);
                }
                if (valid) {
                    uint8_t *d = tsm + (int64_t)cidx[k] * CH;
                    if constexpr (CH == 16) {
                        uint4 o;
                        o.x = signmant4(w[k][0].x, w[k][0].y);
                        o.y = signmant4(w[k][0].z, w[k][0].w);
                        o.z = signmant4(w[k][1].x, w[k][1].y);
                        o.w = signmant4(w[k][1].z, w[k][1].w);
                        __stcs(reinterpret_cast<uint4 *>(d), o);
                    } else {
                        uint2 o;
                        o.x = signmant4(w[k][0].x, w[k][0].y);
                        o.y = signmant4(w[k][0].z, w[k][0].w);
                        __stcs(reinterpret_cast<uint2 *>(d), o);
                    }
                    store_chunk_codes<N, CH>(s_codes + (cidx[k] - slab * kSlabChunks) * CB, g);
                }
            }

            int incl[kCPT];
            const int wtot = warp_scan4(zc, incl);
            if (lane == 0) s_warp_tot[warp] = wtot;
            __syncthreads();
            int wprefix = 0, slab_tot = 0;
#pragma unroll
            for (int i = 0; i < kWarps; ++i) {
                const int t = s_warp_tot[i];
                wprefix += (i < warp) ? t : 0;
                slab_tot += t;
            }

            // escapes: rare, so the raw exponent is re-read from the (cached) source line
#pragma unroll
            for (int k = 0; k < kCPT; ++k) {
                if (zc[k] != 0) {
                    uint8_t *out = tesc + running + wprefix + incl[k] - zc[k];
#pragma unroll
                    for (int q = 0; q < W; ++q) {
                        uint32_t z = zm[k][q];
                        while (z) {
                            const int pos = 31 - __clz(z);
                            z ^= 1u << pos;
                            const int el = q * 8 + 7 - pos / N;
                            const uint32_t e = (cptr[k][el] >> 7) & 0xFFu;
                            *out++ = (uint8_t)e;
                            if (HIST) atomicAdd(&s_hist[e], 1);
                        }
                    }
                }
            }
            running += slab_tot;

            const int slab_chunks = min(kSlabChunks, a.chunks_per_tile - slab * kSlabChunks);
            block_copy_out(tcodes + (int64_t)slab * kSlabChunks * CB, s_codes, slab_chunks * CB);
            __syncthreads();
        }
        if (tid == 0) a.tile_counts[tile] = running;
    }

    if (HIST) {
        // in-window bins: warp sums, then one shared atomic per warp and bin
#pragma unroll
        for (int v = 1; v < (1 << N); ++v) {
            const uint32_t s = __reduce_add_sync(kFull, cnt[v]);
            const int bin = a.left + v;
            if (lane == 0 && s != 0 && bin >= 0 && bin < 256) atomicAdd(&s_hist[bin], (int)s);
        }
        __syncthreads();
        const int hv = s_hist[tid];
        if (hv != 0) atomicAdd(a.hist + tid, hv);
    }

    // The block that finishes last turns the per-tile counts into the per-segment inclusive
    // tile bases and the segment offsets.  No block waits for another.
    __threadfence();
    if (tid == 0) {
        const unsigned ticket = atomicAdd(a.done, 1u);
        s_is_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_is_last) return;
    __threadfence();

    __shared__ long long s_carry;
    __shared__ int s_scan[kWarps];
    if (tid == 0) {
        s_carry = 0;
        a.seg_off[0] = 0;
    }
    __syncthreads();
    for (int64_t base = 0; base < a.n_tiles; base += kThreads) {
        const int64_t t = base + tid;
        const int c = (t < a.n_tiles) ? __ldcg(a.tile_counts + t) : 0;
        int x = c;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int u = __shfl_up_sync(kFull, x, d);
            if (lane >= d) x += u;
        }
        if (lane == 31) s_scan[warp] = x;
        __syncthreads();
        int wp = 0, tot = 0;
#pragma unroll
        for (int i = 0; i < kWarps; ++i) {
            const int v = s_scan[i];
            wp += (i < warp) ? v : 0;
            tot += v;
        }
        const long long incl = s_carry + wp + x;   // inclusive count over the whole call
        if (t < a.n_tiles) {
            // stash the call-wide inclusive count; rebased to the segment below
            a.tile_base[t] = (int32_t)incl;
            if ((t + 1) % a.BH == 0) a.seg_off[(t + 1) / a.BH] = incl;
        }
        __syncthreads();
        if (tid == 0) s_carry += tot;
        __syncthreads();
    }
    __threadfence_block();
    for (int64_t t = tid; t < a.n_tiles; t += kThreads) {
        const int64_t blk = t / a.BH;
        if (blk > 0) a.tile_base[t] -= (int32_t)a.seg_off[blk];
    }
    if (tid == 0) *a.done = 0u;
}

// Gather every tile's escape bytes from its scratch slot into the compact per-segment
// stream: tile t of segment j lands at seg_off[j] + tile_base[t] - count[t].
__global__ void __launch_bounds__(kThreads) k_compact_escapes(const uint8_t *__restrict__ scratch,
                                                               const int32_t *__restrict__ tile_counts,
                                                               const int32_t *__restrict__ tile_base,
                                                               const int64_t *__restrict__ seg_off, int64_t n_tiles,
                                                               int BH, int tile_elems, uint8_t *__restrict__ escapes,
                                                               int64_t capacity, int32_t *status) {
    const int lane = threadIdx.x & 31;
    const int64_t warp_global = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5);
    const int64_t n_warps = (int64_t)gridDim.x * kWarps;
    for (int64_t t = warp_global; t < n_tiles; t += n_warps) {
        const int c = tile_counts[t];
        if (c == 0) continue;
        const int64_t dst = seg_off[t / BH] + tile_base[t] - c;
        if (dst < 0 || dst + c > capacity) {
            if (lane == 0) atomicOr(status, ADACODE_STATUS_ESCAPE_OVERFLOW);
            continue;
        }
        const uint8_t *s = scratch + t * tile_elems;
        for (int i = lane; i < c; i += 32) escapes[dst + i] = s[i];
    }
}

// ---------------------------------------------------------------------------------------
// unpack
// ---------------------------------------------------------------------------------------

struct UnpackCommon {
    int H, BH, seq_tile, D;
    int tile_elems;
    uint16_t *dst;
    int64_t db, dh, ds;
    int32_t *status;
};

// Two bf16 (one 32-bit word) from two sign/mantissa bytes held one per 16-bit lane, two
// exponent codes and the window's left edge replicated in both lanes (left2 = (left & 0xFF)
// * 0x10001).  A code-0 placeholder may wrap inside its own 8-bit field but never leaks
// into the neighbouring element.
__device__ __forceinline__ uint32_t assemble2(uint32_t smlanes, uint32_t c0, uint32_t c1, uint32_t left2) {
    const uint32_t e2 = (__byte_perm(c0, c1, 0x5410) + left2) & 0x00FF00FFu;
    return ((smlanes & 0x00800080u) << 8) | (smlanes & 0x007F007Fu) | (e2 << 7);
}

template <int N, int CH>
__device__ __forceinline__ void unpack_tile(const UnpackCommon &u, const uint8_t *tsm, const uint8_t *tcodes,
                                            const uint8_t *esc, int64_t esc_len, int64_t esc_start, int left,
                                            uint16_t *tdst, uint8_t *s_codes, int *s_warp_tot) {
    constexpr int W = CH / 8;
    constexpr int CB = CH * N / 8;
    constexpr uint32_t kMask = (1u << N) - 1u;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int chunks_per_tile = u.tile_elems / CH;
    const int n_slabs = (chunks_per_tile + kSlabChunks - 1) / kSlabChunks;
    const bool rows_contig = (u.ds == u.D);
    const uint32_t left2 = ((uint32_t)left & 0xFFu) * 0x10001u;
    int64_t running = esc_start;

    for (int slab = 0; slab < n_slabs; ++slab) {
        const int slab_chunks = min(kSlabChunks, chunks_per_tile - slab * kSlabChunks);
        block_copy_in(s_codes, tcodes + (int64_t)slab * kSlabChunks * CB, slab_chunks * CB);

        uint32_t sm[kCPT][CH / 4];
        int cidx[kCPT];
#pragma unroll
        for (int k = 0; k < kCPT; ++k) {
            const int c = slab * kSlabChunks + warp * (kCPT * 32) + k * 32 + lane;
            cidx[k] = c;
            const bool valid = c < chunks_per_tile;
            if constexpr (CH == 16) {
                const uint4 v = valid ? __ldcs(reinterpret_cast<const uint4 *>(tsm + (int64_t)c * CH))
                                      : make_uint4(0, 0, 0, 0);
                sm[k][0] = v.x, sm[k][1] = v.y, sm[k][2] = v.z, sm[k][3] = v.w;
            } else {
                const uint2 v = valid ? __ldcs(reinterpret_cast<const uint2 *>(tsm + (int64_t)c * CH))
                                      : make_uint2(0, 0);
                sm[k][0] = v.x, sm[k][1] = v.y;
            }
        }
        __syncthreads();

        int zc[kCPT];
        uint32_t zm[kCPT][W];
        uint16_t *optr[kCPT];
#pragma unroll
        for (int k = 0; k < kCPT; ++k) {
            const bool valid = cidx[k] < chunks_per_tile;
            uint32_t g[W];
            zc[k] = 0;
#pragma unroll
            for (int q = 0; q < W; ++q) g[q] = 0;
            if (valid) load_chunk_codes<N, CH>(s_codes + (cidx[k] - slab * kSlabChunks) * CB, g);
            const int e0 = cidx[k] * CH;
            int64_t off;
            if (rows_contig) {
                off = e0;
            } else {
                const int row = e0 / u.D;
                off = (int64_t)row * u.ds + (e0 - row * u.D);
            }
            optr[k] = tdst + off;
#pragma unroll
            for (int q = 0; q < W; ++q) {
                zm[k][q] = valid ? zero_slots<N>(g[q]) : 0u;
                zc[k] += __popc(zm[k][q]);
                uint32_t c[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) c[j] = (g[q] >> ((7 - j) * N)) & kMask;
                const uint32_t s0 = sm[k][2 * q], s1 = sm[k][2 * q + 1];
                uint4 o;
                o.x = assemble2(__byte_perm(s0, 0u, 0x4140), c[0], c[1], left2);
                o.y = assemble2(__byte_perm(s0, 0u, 0x4342), c[2], c[3], left2);
                o.z = assemble2(__byte_perm(s1, 0u, 0x4140), c[4], c[5], left2);
                o.w = assemble2(__byte_perm(s1, 0u, 0x4342), c[6], c[7], left2);
                if (valid) __stcs(reinterpret_cast<uint4 *>(optr[k]) + q, o);
            }
        }

        int incl[kCPT];
        const int wtot = warp_scan4(zc, incl);
        if (lane == 0) s_warp_tot[warp] = wtot;
        __syncthreads();
        int wprefix = 0, slab_tot = 0;
#pragma unroll
        for (int i = 0; i < kWarps; ++i) {
            const int t = s_warp_tot[i];
            wprefix += (i < warp) ? t : 0;
            slab_tot += t;
        }

        // escaped elements: patch the exponent field of the 16-bit word just written
#pragma unroll
        for (int k = 0; k < kCPT; ++k) {
            if (zc[k] != 0) {
                int64_t r = running + wprefix + incl[k] - zc[k];
                const uint8_t *smp = tsm + (int64_t)cidx[k] * CH;
#pragma unroll
                for (int q = 0; q < W; ++q) {
                    uint32_t z = zm[k][q];
                    while (z) {
                        const int pos = 31 - __clz(z);
                        z ^= 1u << pos;
                        const int el = q * 8 + 7 - pos / N;
                        uint32_t e = 0;
                        if (r < esc_len) e = esc[r];
                        else atomicOr(u.status, ADACODE_STATUS_ESCAPE_UNDERRUN);
                        ++r;
                        const uint32_t s = smp[el];
                        optr[k][el] = (uint16_t)(((s & 0x80u) << 8) | (s & 0x7Fu) | (e << 7));
                    }
                }
            }
        }
        running += slab_tot;
        __syncthreads();   // s_codes and s_warp_tot are reused by the next slab
    }
}

template <int CH>
__device__ __forceinline__ void unpack_dispatch(int nbits, const UnpackCommon &u, const uint8_t *tsm,
                                                const uint8_t *tcodes, const uint8_t *esc, int64_t esc_len,
                                                int64_t esc_start, int left, uint16_t *tdst, uint8_t *s_codes,
                                                int *s_warp_tot) {
    switch (nbits) {
        case 1: unpack_tile<1, CH>(u, tsm, tcodes, esc, esc_len, esc_start, left, tdst, s_codes, s_warp_tot); break;
        case 2: unpack_tile<2, CH>(u, tsm, tcodes, esc, esc_len, esc_start, left, tdst, s_codes, s_warp_tot); break;
        case 3: unpack_tile<3, CH>(u, tsm, tcodes, esc, esc_len, esc_start, left, tdst, s_codes, s_warp_tot); break;
        default: unpack_tile<4, CH>(u, tsm, tcodes, esc, esc_len, esc_start, left, tdst, s_codes, s_warp_tot); break;
    }
}

// Segments that share one window, laid out as adacode_pack_tiles writes them.
template <int CH>
__global__ void __launch_bounds__(kThreads) k_unpack_uniform(const UnpackCommon u, const uint8_t *sign_mant,
                                                             const uint8_t *codes, const uint8_t *escapes,
                                                             int64_t escapes_len, const int32_t *tile_base,
                                                             const int64_t *seg_off, int64_t n_tiles, int left,
                                                             int nbits) {
    __shared__ __align__(16) uint8_t s_codes[kSlabChunks * CH * 4 / 8];
    __shared__ int s_warp_tot[kWarps];
    const int tile_code_bytes = u.tile_elems * nbits / 8;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t blk = tile / u.BH;
        const int bh = (int)(tile - blk * u.BH);
        const int b = bh / u.H, h = bh - b * u.H;
        const int64_t seg_start = seg_off ? seg_off[blk] : 0;
        const int64_t esc_start = seg_start + (bh > 0 ? tile_base[tile - 1] : 0);
        uint16_t *tdst = u.dst + (int64_t)b * u.db + (int64_t)h * u.dh + blk * u.seq_tile * u.ds;
        unpack_dispatch<CH>(nbits, u, sign_mant + tile * u.tile_elems, codes + tile * tile_code_bytes, escapes,
                            escapes_len, esc_start, left, tdst, s_codes, s_warp_tot);
    }
}

// Segments described one by one (mixed windows and code lengths).
template <int CH>
__global__ void __launch_bounds__(kThreads) k_unpack_segments(const UnpackCommon u,
                                                              const adacode_segment *__restrict__ segs,
                                                              int64_t n_tiles) {
    __shared__ __align__(16) uint8_t s_codes[kSlabChunks * CH * 4 / 8];
    __shared__ int s_warp_tot[kWarps];
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t si = tile / u.BH;
        const int bh = (int)(tile - si * u.BH);
        const int b = bh / u.H, h = bh - b * u.H;
        const adacode_segment sg = segs[si];
        const int tile_code_bytes = u.tile_elems * sg.nbits / 8;
        const int64_t esc_start = bh > 0 ? sg.tile_base[bh - 1] : 0;
        uint16_t *tdst = u.dst + (int64_t)b * u.db + (int64_t)h * u.dh + sg.dst_seq_offset * u.ds;
        unpack_dispatch<CH>(sg.nbits, u, sg.sign_mant + (int64_t)bh * u.tile_elems,
                            sg.codes + (int64_t)bh * tile_code_bytes, sg.escapes, sg.escapes_len, esc_start,
                            sg.left, tdst, s_codes, s_warp_tot);
    }
}

// ---------------------------------------------------------------------------------------
// histogram and adjuster
// ---------------------------------------------------------------------------------------

__global__ void __launch_bounds__(kThreads) k_hist(const uint16_t *__restrict__ src, int64_t sb, int64_t sh,
                                                   int64_t ss, int H, int S, int D, int64_t n_rows,
                                                   int32_t *__restrict__ hist) {
    __shared__ int s_hist[kWarps][256];
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < kWarps * 256; i += kThreads) (&s_hist[0][0])[i] = 0;
    __syncthreads();
    const int vec_per_row = D / 8;
    const int64_t n_vec = n_rows * vec_per_row;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + tid; i < n_vec; i += (int64_t)gridDim.x * kThreads) {
        const int64_t row = i / vec_per_row;
        const int col = (int)(i - row * vec_per_row) * 8;
        const int64_t bh = row / S;
        const int s = (int)(row - bh * S);
        const int b = (int)(bh / H), h = (int)(bh - (int64_t)b * H);
        const uint4 v = *reinterpret_cast<const uint4 *>(src + b * sb + h * sh + s * ss + col);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            atomicAdd(&s_hist[warp][(w[q] >> 7) & 0xFFu], 1);
            atomicAdd(&s_hist[warp][(w[q] >> 23) & 0xFFu], 1);
        }
    }
    __syncthreads();
    int total = 0;
#pragma unroll
    for (int i = 0; i < kWarps; ++i) total += s_hist[i][tid];
    if (total != 0) atomicAdd(hist + tid, total);
}

// One warp per histogram: fifteen rounds of "largest remaining count, lowest bin on ties"
// reproduce a stable descending sort's first fifteen entries.
__global__ void k_choose_params(const int32_t *__restrict__ hists, int n_hists, int32_t *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int hidx = blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
    if (hidx >= n_hists) return;
    const int32_t *hist = hists + (int64_t)hidx * 256;
    long long v[8];
    long long total = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        v[i] = hist[i * 32 + lane];
        total += v[i];
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) total += __shfl_xor_sync(kFull, total, d);

    long long covered = 0;
    int max_bin = -1;
    long long best = total * 8;
    int best_n = 0, best_right = -1;
    for (int k = 1; k <= 15; ++k) {
        // key = count * 256 + (255 - bin): larger count first, then lower bin
        long long key = -1;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (v[i] >= 0) {
                const long long cand = v[i] * 256 + (255 - (i * 32 + lane));
                key = cand > key ? cand : key;
            }
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const long long o = __shfl_xor_sync(kFull, key, d);
            key = o > key ? o : key;
        }
        const int bin = 255 - (int)(key & 255);
        covered += key >> 8;
        max_bin = bin > max_bin ? bin : max_bin;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (i * 32 + lane == bin) v[i] = -1;
        if (k == 3 || k == 7 || k == 15) {
            const int n = (k == 3) ? 2 : (k == 7 ? 3 : 4);
            const long long cost = total * n + (total - covered) * 8;
            if (cost < best) {
                best = cost;
                best_n = n;
                best_right = max_bin;
            }
        }
    }
    if (lane == 0) {
        out[2 * hidx] = best_right;
        out[2 * hidx + 1] = best_n;
    }
}

#include "adacode_pipeline.cuh"

void stable_order_desc(const int64_t *hist, int *order) {
    for (int i = 0; i < 256; ++i) order[i] = i;
    for (int i = 1; i < 256; ++i) {
        const int idx = order[i];
        int j = i - 1;
        while (j >= 0 && hist[order[j]] < hist[idx]) {
            order[j + 1] = order[j];
            --j;
        }
        order[j + 1] = idx;
    }
}

int choose_host(const int64_t *hist, int n_lo, int n_hi, bool escape_slot, int *right, int *nbits) {
    if (!hist || !right || !nbits) return ADACODE_ERR_INVALID_ARG;
    int order[256];
    stable_order_desc(hist, order);
    int64_t total = 0;
    for (int i = 0; i < 256; ++i) total += hist[i];
    int64_t best = total * 8;
    int best_n = 0, best_right = -1;
    for (int n = n_lo; n <= n_hi; ++n) {
        const int space = (1 << n) - (escape_slot ? 1 : 0);
        int64_t covered = 0;
        int mx = -1;
        for (int k = 0; k < space && k < 256; ++k) {
            covered += hist[order[k]];
            mx = order[k] > mx ? order[k] : mx;
        }
        const int64_t cost = total * n + (total - covered) * 8;
        if (cost < best) {
            best = cost;
            best_n = n;
            best_right = mx;
        }
    }
    if (best_n == 0) return ADACODE_ERR_NO_CANDIDATE;
    *right = best_right;
    *nbits = best_n;
    return ADACODE_OK;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
size_t unit_counts_bytes(int64_t n_tiles, int64_t tile_elems) {
    return align_up((size_t)n_tiles * (size_t)(tile_elems / 128 + 1) * 4, 256);
}

// Layout of the pack scratch: [completion counter, 256 B][tile_counts int32][unit_counts int32]
// [block offsets int64, one more than blocks][escape slots, tile_elems bytes per tile].
struct PackScratch {
    unsigned int *done;
    int32_t *tile_counts;
    int32_t *unit_counts;
    int64_t *blk_off;
    uint8_t *esc;
    size_t bytes;
};

PackScratch carve_pack_scratch(void *workspace, int64_t n_tiles, int64_t tile_elems) {
    uint8_t *ws = (uint8_t *)workspace;
    PackScratch p;
    size_t off = 0;
    p.done = (unsigned int *)(ws + off);
    off += 256;
    p.tile_counts = (int32_t *)(ws + off);
    off += align_up((size_t)n_tiles * 4, 256);
    p.unit_counts = (int32_t *)(ws + off);
    off += unit_counts_bytes(n_tiles, tile_elems);
    p.blk_off = (int64_t *)(ws + off);
    off += align_up((size_t)(n_tiles + 2) * 8, 256);     // a launch has at most as many blocks as tiles
    p.esc = ws + off;
    off += (size_t)n_tiles * (size_t)tile_elems;
    p.bytes = off;
    return p;
}

int grid_for(int64_t n_tiles, int ctas_per_sm) {
    const int64_t cap = (int64_t)sm_count() * ctas_per_sm;
    return (int)(n_tiles < cap ? n_tiles : cap);
}


bool pipeline_enabled() {
    static int cached = -1;
    if (cached < 0) {
        const char *e = getenv("ADACODE_DISABLE_PIPELINE");
        cached = (e && e[0] == '1') ? 0 : 1;
    }
    return cached == 1;
}

// The pipelined kernels move whole units with bulk copies: 16-byte aligned planes, head_dim a
// multiple of 16 and at most 2048, token rows in multiples of 8.
bool pipeline_shape_ok(int seq_tile, int D) { return D % 16 == 0 && D <= 2048 && seq_tile % 8 == 0; }

template <typename Kernel>
int ensure_dynamic_smem(Kernel kernel, size_t bytes) {
    // per device and kernel; the attribute call is cheap but not free
    static thread_local const void *last_kernel[16] = {nullptr};
    int dev = 0;
    ADACODE_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 16 && last_kernel[dev] == (const void *)kernel) return ADACODE_OK;
    ADACODE_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    if (dev >= 0 && dev < 16) last_kernel[dev] = (const void *)kernel;
    return ADACODE_OK;
}

// bound of the on-chip waits and the testing aid of adacode_debug_set_wait_limit
uint32_t g_poll_limit = kMaxPolls;
int g_withhold_unit = -1;

// Launch as a programmatic dependent of whatever precedes it in the stream: the kernel may be set up
// (barriers, tables in shared memory) while its predecessor's last CTAs still run; it executes
// griddepcontrol.wait before it touches global memory.
template <typename Kernel, typename Args>
int launch_dependent(Kernel kernel, dim3 grid, int threads, size_t smem, cudaStream_t st, const Args &args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid, cfg.blockDim = dim3(threads), cfg.dynamicSmemBytes = smem, cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    ADACODE_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, args));
    return ADACODE_OK;
}

template <class G>
int launch_unpack_geom(const UnpackJobsArgs &ja, cudaStream_t st) {
    int rc = ensure_dynamic_smem(k_unpack_pipe<G>, sizeof(UnpackSmemT<G>));
    if (rc != ADACODE_OK) return rc;
    const int grid = grid_for(ja.tile0[ja.n_jobs], G::kCtasPerSm);
    return launch_dependent(k_unpack_pipe<G>, dim3(grid), G::kThreads, sizeof(UnpackSmemT<G>), st, ja);
}

// ADACODE_UNPACK_GEOMETRY=wide keeps the unpack kernel on the 16-warp geometry (for comparisons)
bool unpack_prefers_wide() {
    static int cached = -1;
    if (cached < 0) {
        const char *e = getenv("ADACODE_UNPACK_GEOMETRY");
        cached = (e && strcmp(e, "wide") == 0) ? 1 : 0;
    }
    return cached == 1;
}

int launch_unpack_pipe(UnpackJobsArgs &ja, cudaStream_t st) {
    ja.poll_limit = g_poll_limit;
    ja.withhold_unit = g_withhold_unit;
    // a unit holds at least eight token rows: the narrow geometry takes head_dim up to 1024
    const bool narrow = ja.job[0].D <= NarrowGeom::kUnit / 8 && !unpack_prefers_wide();
    return narrow ? launch_unpack_geom<NarrowGeom>(ja, st) : launch_unpack_geom<WideGeom>(ja, st);
}

int launch_unpack_pipe(const UnpackPipeArgs &a, cudaStream_t st) {
    UnpackJobsArgs ja;
    ja.job[0] = a;
    ja.tile0[0] = 0, ja.tile0[1] = a.n_tiles;
    ja.n_jobs = 1;
    return launch_unpack_pipe(ja, st);
}

template <class G, typename Kernel>
int launch_pack_kernel(Kernel kernel, const PackPipeArgs &pa, cudaStream_t st) {
    int rc = ensure_dynamic_smem(kernel, sizeof(PackSmemT<G>));
    if (rc != ADACODE_OK) return rc;
    return launch_dependent(kernel, dim3(grid_for(pa.n_tiles, G::kCtasPerSm)), G::kThreads, sizeof(PackSmemT<G>), st, pa);
}

template <int N, class G>
int launch_pack_pipe_n(const PackPipeArgs &pa, bool hist, cudaStream_t st) {
    return hist ? launch_pack_kernel<G>(k_pack_pipe<N, true, G>, pa, st)
                : launch_pack_kernel<G>(k_pack_pipe<N, false, G>, pa, st);
}

// The pack kernel takes the narrow geometry where a unit of the wide one would stay half empty
// (tiles of at most 8192 elements, e.g. 128 tokens of a 64-wide head).
// ADACODE_PACK_GEOMETRY=wide|narrow overrides the choice where the shape allows it (for comparisons).
bool pack_takes_narrow(int seq_tile, int D) {
    static int forced = -1;
    if (forced < 0) {
        const char *e = getenv("ADACODE_PACK_GEOMETRY");
        forced = !e ? 0 : strcmp(e, "wide") == 0 ? 1 : strcmp(e, "narrow") == 0 ? 2 : 0;
    }
    if (D > NarrowGeom::kUnit / 8) return false;      // a unit holds at least eight token rows
    if (forced != 0) return forced == 2;
    return unit_rows_for<WideGeom::kUnit>(seq_tile, D) * D <= NarrowGeom::kUnit;
}

// Pipelined pack of all jobs of `pa` with one pack launch and one compaction launch.
int launch_pack_pipe(PackPipeArgs &pa, int nbits, cudaStream_t st) {
    const bool narrow = pack_takes_narrow(pa.seq_tile, pa.D);
    pa.unit_rows = narrow ? unit_rows_for<NarrowGeom::kUnit>(pa.seq_tile, pa.D)
                          : unit_rows_for<WideGeom::kUnit>(pa.seq_tile, pa.D);
    pa.units_per_tile = (pa.seq_tile + pa.unit_rows - 1) / pa.unit_rows;
    bool hist = false;
    int max_blocks = 0;
    for (int j = 0; j < pa.n_jobs; ++j) {
        hist = hist || pa.job[j].hist != nullptr;
        max_blocks = pa.job[j].n_blocks > max_blocks ? pa.job[j].n_blocks : max_blocks;
    }
    int rc;
    switch (nbits + (narrow ? 4 : 0)) {
        case 1: rc = launch_pack_pipe_n<1, WideGeom>(pa, hist, st); break;
        case 2: rc = launch_pack_pipe_n<2, WideGeom>(pa, hist, st); break;
        case 3: rc = launch_pack_pipe_n<3, WideGeom>(pa, hist, st); break;
        case 4: rc = launch_pack_pipe_n<4, WideGeom>(pa, hist, st); break;
        case 5: rc = launch_pack_pipe_n<1, NarrowGeom>(pa, hist, st); break;
        case 6: rc = launch_pack_pipe_n<2, NarrowGeom>(pa, hist, st); break;
        case 7: rc = launch_pack_pipe_n<3, NarrowGeom>(pa, hist, st); break;
        default: rc = launch_pack_pipe_n<4, NarrowGeom>(pa, hist, st); break;
    }
    if (rc != ADACODE_OK) return rc;
    // one warp per tile; few enough CTAs that the final per-bin atomics of the histogram stay cheap
    const int64_t job_tiles = (int64_t)max_blocks * pa.BH;
    const int64_t want = (job_tiles + kWarps - 1) / kWarps;
    const int64_t cap = ((int64_t)sm_count() * 4 + pa.n_jobs - 1) / pa.n_jobs;
    const dim3 cgrid((unsigned)(want < cap ? want : cap), (unsigned)pa.n_jobs);
    // (a programmatic dependent of the pack kernel: it is set up, and clears its histogram copies, while
    // the pack kernel's last CTAs still run)
    return hist ? launch_dependent(k_compact_units<true>, cgrid, kThreads, 0, st, pa)
                : launch_dependent(k_compact_units<false>, cgrid, kThreads, 0, st, pa);
}

template <int N, int CH>
void launch_pack(const PackArgs &a, int grid, cudaStream_t st) {
    if (a.hist) k_pack<N, CH, true><<<grid, kThreads, 0, st>>>(a);
    else k_pack<N, CH, false><<<grid, kThreads, 0, st>>>(a);
}

// Word-wise copy of a small device buffer into host memory that the device can address (pinned
// memory under unified addressing); one CTA.
__global__ void k_copy_to_host(const uint32_t *__restrict__ src, uint32_t *dst, size_t words) {
    for (size_t i = threadIdx.x; i < words; i += blockDim.x) dst[i] = src[i];
    __threadfence_system();
}

}  // namespace

// ---------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------

extern "C" {

int adacode_version(void) { return 100; }

const char *adacode_strerror(int code) {
    switch (code) {
        case ADACODE_OK: return "ok";
        case ADACODE_ERR_INVALID_ARG: return "invalid argument";
        case ADACODE_ERR_CUDA: return "CUDA runtime error";
        case ADACODE_ERR_WORKSPACE: return "workspace too small";
        case ADACODE_ERR_NO_CANDIDATE: return "no code length beats 8 bits per exponent";
        case ADACODE_ERR_TOO_LARGE: return "call covers 2**31 elements or more";
        default: return "unknown adacode error";
    }
}

const char *adacode_last_cuda_error(void) { return g_last_cuda_error; }

int adacode_copy_to_host(const void *src_dev, void *dst_host_pinned, size_t bytes, void *stream) {
    if (bytes == 0) return ADACODE_OK;
    if (!src_dev || !dst_host_pinned || (bytes & 3) != 0 || (((uintptr_t)src_dev | (uintptr_t)dst_host_pinned) & 3) != 0)
        return ADACODE_ERR_INVALID_ARG;
    if (bytes > (1u << 20)) return ADACODE_ERR_TOO_LARGE;
    cudaPointerAttributes attr;
    ADACODE_CUDA_TRY(cudaPointerGetAttributes(&attr, dst_host_pinned));
    // only page-locked host memory that this device can address; anything else is refused, not tried
    if (attr.type != cudaMemoryTypeHost || attr.devicePointer == nullptr) return ADACODE_ERR_INVALID_ARG;
    k_copy_to_host<<<1, 256, 0, (cudaStream_t)stream>>>((const uint32_t *)src_dev, (uint32_t *)attr.devicePointer,
                                                       bytes / 4);
    ADACODE_CUDA_TRY(cudaGetLastError());
    return ADACODE_OK;
}

size_t adacode_pack_workspace_bytes(int64_t n_tiles, int64_t tile_elems) {
    if (n_tiles <= 0 || tile_elems <= 0) return 256;
    // a tile has at most tile_elems / 128 units (a unit is at least 8 rows of at least 16 elements)
    return carve_pack_scratch(nullptr, n_tiles, tile_elems).bytes;
}

}  // extern "C"

namespace {

// The direct (not pipelined) kernels, one job: shapes the bulk-copy pipeline does not take.
int pack_direct(const adacode_pack_job &jb, int B, int H, int seq_tile, int D, int nbits, const PackScratch &sc,
                int32_t *status, cudaStream_t st) {
    const int64_t n_tiles = (int64_t)B * H * jb.n_blocks;
    const int64_t tile_elems = (int64_t)seq_tile * D;
    const int CH = (D % 16 == 0) ? 16 : 8;
    PackArgs a;
    a.src = (const uint16_t *)jb.src_bf16;
    a.sb = jb.stride_b, a.sh = jb.stride_h, a.ss = jb.stride_s;
    a.H = H, a.BH = B * H, a.seq_tile = seq_tile, a.D = D;
    a.left = jb.right - (1 << nbits) + 1;
    a.n_tiles = n_tiles;
    a.tile_elems = (int)tile_elems;
    a.chunks_per_tile = (int)(tile_elems / CH);
    a.tile_code_bytes = (int)(tile_elems * nbits / 8);
    a.sign_mant = jb.sign_mant;
    a.codes = jb.codes;
    a.done = sc.done;
    a.tile_counts = sc.tile_counts;
    a.esc_scratch = sc.esc;
    a.tile_base = jb.tile_base;
    a.seg_off = jb.seg_escape_offsets;
    a.n_blocks = jb.n_blocks;
    a.hist = jb.hist256;
    const int grid = grid_for(n_tiles, 4);
    if (CH == 16) {
        switch (nbits) {
            case 1: launch_pack<1, 16>(a, grid, st); break;
            case 2: launch_pack<2, 16>(a, grid, st); break;
            case 3: launch_pack<3, 16>(a, grid, st); break;
            default: launch_pack<4, 16>(a, grid, st); break;
        }
    } else {
        switch (nbits) {
            case 1: launch_pack<1, 8>(a, grid, st); break;
            case 2: launch_pack<2, 8>(a, grid, st); break;
            case 3: launch_pack<3, 8>(a, grid, st); break;
            default: launch_pack<4, 8>(a, grid, st); break;
        }
    }
    ADACODE_CUDA_TRY(cudaGetLastError());
    const int64_t want = (n_tiles + kWarps - 1) / kWarps;
    const int64_t cap = (int64_t)sm_count() * 4;
    k_compact_escapes<<<(int)(want < cap ? want : cap), kThreads, 0, st>>>(
        a.esc_scratch, a.tile_counts, jb.tile_base, jb.seg_escape_offsets, n_tiles, a.BH, a.tile_elems, jb.escapes,
        jb.escapes_capacity, status);
    ADACODE_CUDA_TRY(cudaGetLastError());
    return ADACODE_OK;
}

int pack_jobs_impl(const adacode_pack_job *jobs, int n_jobs, int B, int H, int seq_tile, int D, int nbits,
                   void *workspace, size_t workspace_bytes, int32_t *status, cudaStream_t st) {
    if (n_jobs < 0 || n_jobs > kMaxJobs || (n_jobs > 0 && !jobs)) return ADACODE_ERR_INVALID_ARG;
    if (B < 0 || H < 0 || seq_tile <= 0 || D <= 0) return ADACODE_ERR_INVALID_ARG;
    if (nbits < 1 || nbits > 4 || D % 8 != 0 || !status) return ADACODE_ERR_INVALID_ARG;
    const int64_t tile_elems = (int64_t)seq_tile * D;
    const int64_t BH = (int64_t)B * H;
    int64_t n_tiles = 0, max_job_tiles = 0;
    for (int j = 0; j < n_jobs; ++j) {
        const adacode_pack_job &jb = jobs[j];
        if (jb.n_blocks < 0 || !jb.seg_escape_offsets || jb.escapes_capacity < 0) return ADACODE_ERR_INVALID_ARG;
        const int64_t jt = BH * jb.n_blocks;
        if (jt == 0) continue;
        if (!jb.src_bf16 || !jb.sign_mant || !jb.codes || !jb.tile_base || (!jb.escapes && jb.escapes_capacity > 0))
            return ADACODE_ERR_INVALID_ARG;
        if ((((uintptr_t)jb.src_bf16 | (uintptr_t)jb.sign_mant | (uintptr_t)jb.codes) & 15) != 0)
            return ADACODE_ERR_INVALID_ARG;
        if ((jb.stride_b | jb.stride_h | jb.stride_s) & 7) return ADACODE_ERR_INVALID_ARG;
        n_tiles += jt;
        max_job_tiles = jt > max_job_tiles ? jt : max_job_tiles;
    }
    for (int j = 0; j < n_jobs; ++j)
        if (BH * jobs[j].n_blocks == 0)
            ADACODE_CUDA_TRY(cudaMemsetAsync(jobs[j].seg_escape_offsets, 0,
                                             sizeof(int64_t) * (size_t)(jobs[j].n_blocks + 1), st));
    if (n_tiles == 0) return ADACODE_OK;
    if (n_tiles * tile_elems >= (1ll << 31)) return ADACODE_ERR_TOO_LARGE;
    if (!workspace || ((uintptr_t)workspace & 15) != 0) return ADACODE_ERR_INVALID_ARG;

    // (the pipelined kernel's unit bookkeeping is 32-bit: keep tiles below 2**24 elements)
    if (pipeline_enabled() && pipeline_shape_ok(seq_tile, D) && tile_elems <= (1 << 24)) {
        if (workspace_bytes < adacode_pack_workspace_bytes(n_tiles, tile_elems)) return ADACODE_ERR_WORKSPACE;
        const PackScratch sc = carve_pack_scratch(workspace, n_tiles, tile_elems);
        PackPipeArgs pa;
        memset(&pa, 0, sizeof(pa));
        int64_t tile0 = 0;
        int blk0 = 0, n = 0;
        for (int j = 0; j < n_jobs; ++j) {
            const adacode_pack_job &jb = jobs[j];
            if (BH * jb.n_blocks == 0) continue;
            PackJob &d = pa.job[n++];
            d.src = (const uint16_t *)jb.src_bf16;
            d.sb = jb.stride_b, d.sh = jb.stride_h, d.ss = jb.stride_s;
            d.sign_mant = jb.sign_mant, d.codes = jb.codes, d.escapes = jb.escapes;
            d.capacity = jb.escapes_capacity;
            d.tile_base = jb.tile_base, d.seg_off = jb.seg_escape_offsets, d.hist = jb.hist256;
            d.tile0 = tile0, d.blk0 = blk0, d.n_blocks = jb.n_blocks;
            d.left = jb.right - (1 << nbits) + 1;
            tile0 += BH * jb.n_blocks;
            blk0 += jb.n_blocks;
        }
        pa.n_jobs = n;
        pa.H = H, pa.BH = (int)BH, pa.seq_tile = seq_tile, pa.D = D, pa.tile_elems = (int)tile_elems;
        pa.n_tiles = n_tiles;
        pa.esc_scratch = sc.esc, pa.tile_counts = sc.tile_counts, pa.unit_counts = sc.unit_counts;
        pa.blk_off = sc.blk_off, pa.done = sc.done;
        pa.status = status;
        pa.poll_limit = g_poll_limit;
        return launch_pack_pipe(pa, nbits, st);
    }
    if (workspace_bytes < adacode_pack_workspace_bytes(max_job_tiles, tile_elems)) return ADACODE_ERR_WORKSPACE;
    const PackScratch sc = carve_pack_scratch(workspace, max_job_tiles, tile_elems);
    for (int j = 0; j < n_jobs; ++j) {
        if (BH * jobs[j].n_blocks == 0) continue;
        const int rc = pack_direct(jobs[j], B, H, seq_tile, D, nbits, sc, status, st);
        if (rc != ADACODE_OK) return rc;
    }
    return ADACODE_OK;
}

}  // namespace

extern "C" {

int adacode_pack_jobs(const adacode_pack_job *jobs, int n_jobs, int B, int H, int seq_tile, int D, int nbits,
                      void *workspace, size_t workspace_bytes, int32_t *status, void *stream) {
    return pack_jobs_impl(jobs, n_jobs, B, H, seq_tile, D, nbits, workspace, workspace_bytes, status,
                          (cudaStream_t)stream);
}

int adacode_max_jobs(void) { return kMaxJobs; }

int adacode_debug_set_wait_limit(unsigned int polls, int withhold_unit) {
    g_poll_limit = polls == 0 ? kMaxPolls : polls;
    g_withhold_unit = withhold_unit;
    return ADACODE_OK;
}

int adacode_pack_tiles(const void *src_bf16, int64_t stride_b, int64_t stride_h, int64_t stride_s, int B, int H,
                       int n_blocks, int seq_tile, int D, int right, int nbits, uint8_t *sign_mant, uint8_t *codes,
                       uint8_t *escapes, int64_t escapes_capacity, int32_t *tile_base, int64_t *seg_escape_offsets,
                       int32_t *hist256, void *workspace, size_t workspace_bytes, int32_t *status, void *stream) {
    adacode_pack_job jb;
    jb.src_bf16 = src_bf16;
    jb.stride_b = stride_b, jb.stride_h = stride_h, jb.stride_s = stride_s;
    jb.n_blocks = n_blocks, jb.right = right;
    jb.sign_mant = sign_mant, jb.codes = codes, jb.escapes = escapes;
    jb.escapes_capacity = escapes_capacity;
    jb.tile_base = tile_base, jb.seg_escape_offsets = seg_escape_offsets, jb.hist256 = hist256;
    return pack_jobs_impl(&jb, 1, B, H, seq_tile, D, nbits, workspace, workspace_bytes, status, (cudaStream_t)stream);
}

static int check_unpack_common(int B, int H, int seq_tile, int D, const void *dst, int64_t db, int64_t dh,
                               int64_t ds, const int32_t *status) {
    if (B < 0 || H < 0 || seq_tile <= 0 || D <= 0 || D % 8 != 0) return ADACODE_ERR_INVALID_ARG;
    if (!dst || !status) return ADACODE_ERR_INVALID_ARG;
    if (((uintptr_t)dst & 15) != 0 || ((db | dh | ds) & 7)) return ADACODE_ERR_INVALID_ARG;
    return ADACODE_OK;
}

int adacode_unpack_tiles(const uint8_t *sign_mant, const uint8_t *codes, const uint8_t *escapes, int64_t escapes_len,
                         const int32_t *tile_base, const int64_t *seg_escape_offsets, int B, int H, int n_blocks,
                         int seq_tile, int D, int left, int nbits, void *dst_bf16, int64_t dstride_b,
                         int64_t dstride_h, int64_t dstride_s, int32_t *status, void *stream) {
    if (n_blocks < 0 || nbits < 1 || nbits > 4) return ADACODE_ERR_INVALID_ARG;
    const int64_t n_tiles = (int64_t)B * H * n_blocks;
    if (n_tiles == 0) return ADACODE_OK;
    int rc = check_unpack_common(B, H, seq_tile, D, dst_bf16, dstride_b, dstride_h, dstride_s, status);
    if (rc != ADACODE_OK) return rc;
    if (!sign_mant || !codes || !tile_base || (n_blocks > 1 && !seg_escape_offsets)) return ADACODE_ERR_INVALID_ARG;
    if ((((uintptr_t)sign_mant | (uintptr_t)codes) & 15) != 0) return ADACODE_ERR_INVALID_ARG;
    if (n_tiles * (int64_t)seq_tile * D >= (1ll << 31)) return ADACODE_ERR_TOO_LARGE;
    UnpackCommon u;
    u.H = H, u.BH = B * H, u.seq_tile = seq_tile, u.D = D;
    u.tile_elems = seq_tile * D;
    u.dst = (uint16_t *)dst_bf16;
    u.db = dstride_b, u.dh = dstride_h, u.ds = dstride_s;
    u.status = status;
    cudaStream_t st = (cudaStream_t)stream;
    if (pipeline_enabled() && pipeline_shape_ok(seq_tile, D)) {
        UnpackPipeArgs pa;
        pa.sign_mant = sign_mant, pa.codes = codes, pa.escapes = escapes, pa.escapes_len = escapes_len;
        pa.tile_base = tile_base, pa.seg_off = seg_escape_offsets, pa.left = left, pa.nbits = nbits;
        pa.tb_stride = 1, pa.tb_before = 0;
        pa.seg = nullptr;
        pa.H = H, pa.BH = B * H, pa.seq_tile = seq_tile, pa.D = D, pa.tile_elems = seq_tile * D;
        pa.n_tiles = n_tiles, pa.dst = (uint16_t *)dst_bf16;
        pa.db = dstride_b, pa.dh = dstride_h, pa.ds = dstride_s, pa.status = status;
        return launch_unpack_pipe(pa, st);
    }
    const int grid = grid_for(n_tiles, 6);
    if (D % 16 == 0)
        k_unpack_uniform<16><<<grid, kThreads, 0, st>>>(u, sign_mant, codes, escapes, escapes_len, tile_base,
                                                        seg_escape_offsets, n_tiles, left, nbits);
    else
        k_unpack_uniform<8><<<grid, kThreads, 0, st>>>(u, sign_mant, codes, escapes, escapes_len, tile_base,
                                                       seg_escape_offsets, n_tiles, left, nbits);
    ADACODE_CUDA_TRY(cudaGetLastError());
    return ADACODE_OK;
}

int adacode_unpack_segments(const adacode_segment *segments_dev, int n_segments, int B, int H, int seq_tile, int D,
                            void *dst_bf16, int64_t dstride_b, int64_t dstride_h, int64_t dstride_s, int32_t *status,
                            void *stream) {
    if (n_segments < 0) return ADACODE_ERR_INVALID_ARG;
    const int64_t n_tiles = (int64_t)B * H * n_segments;
    if (n_tiles == 0) return ADACODE_OK;
    int rc = check_unpack_common(B, H, seq_tile, D, dst_bf16, dstride_b, dstride_h, dstride_s, status);
    if (rc != ADACODE_OK) return rc;
    if (!segments_dev) return ADACODE_ERR_INVALID_ARG;
    UnpackCommon u;
    u.H = H, u.BH = B * H, u.seq_tile = seq_tile, u.D = D;
    u.tile_elems = seq_tile * D;
    u.dst = (uint16_t *)dst_bf16;
    u.db = dstride_b, u.dh = dstride_h, u.ds = dstride_s;
    u.status = status;
    cudaStream_t st = (cudaStream_t)stream;
    if (pipeline_enabled() && pipeline_shape_ok(seq_tile, D)) {
        UnpackPipeArgs pa;
        pa.sign_mant = nullptr, pa.codes = nullptr, pa.escapes = nullptr, pa.escapes_len = 0;
        pa.tile_base = nullptr, pa.seg_off = nullptr, pa.left = 0, pa.nbits = 0;
        pa.tb_stride = 1, pa.tb_before = 0;
        pa.seg = segments_dev;
        pa.H = H, pa.BH = B * H, pa.seq_tile = seq_tile, pa.D = D, pa.tile_elems = seq_tile * D;
        pa.n_tiles = n_tiles, pa.dst = (uint16_t *)dst_bf16;
        pa.db = dstride_b, pa.dh = dstride_h, pa.ds = dstride_s, pa.status = status;
        return launch_unpack_pipe(pa, st);
    }
    const int grid = grid_for(n_tiles, 6);
    if (D % 16 == 0) k_unpack_segments<16><<<grid, kThreads, 0, st>>>(u, segments_dev, n_tiles);
    else k_unpack_segments<8><<<grid, kThreads, 0, st>>>(u, segments_dev, n_tiles);
    ADACODE_CUDA_TRY(cudaGetLastError());
    return ADACODE_OK;
}

int adacode_flat_block_elems(int nbits) {
    static const int gaps[4] = {8, 4, 8, 2};
    return (nbits < 1 || nbits > 4) ? 0 : 128 * gaps[nbits - 1];
}

int adacode_unpack_flat(const uint8_t *sign_mant, const uint8_t *codes, const uint8_t *escapes, int64_t escapes_len,
                        const int32_t *block_base, int64_t n_elems, int left, int nbits, void *dst_bf16,
                        int32_t *status, void *stream) {
    const int be = adacode_flat_block_elems(nbits);
    if (be == 0 || n_elems < 0 || n_elems % be != 0 || !status) return ADACODE_ERR_INVALID_ARG;
    if (n_elems == 0) return ADACODE_OK;
    if (n_elems >= (1ll << 31)) return ADACODE_ERR_TOO_LARGE;
    if (!sign_mant || !codes || !block_base || !dst_bf16) return ADACODE_ERR_INVALID_ARG;
    if ((((uintptr_t)sign_mant | (uintptr_t)codes | (uintptr_t)dst_bf16) & 15) != 0) return ADACODE_ERR_INVALID_ARG;
    if (!pipeline_enabled()) return ADACODE_ERR_INVALID_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    // the bulk of the tensor as 128 x 128 tiles whose escape base is every (16384 / be)-th block base,
    // the rest (fewer than 16384 elements) block by block
    const int64_t big = 128 * 128;
    const int64_t n_big = n_elems / big;
    const int64_t n_main = n_big * big;
    UnpackPipeArgs pa;
    memset(&pa, 0, sizeof(pa));
    pa.escapes = escapes, pa.escapes_len = escapes_len, pa.seg_off = nullptr, pa.left = left, pa.nbits = nbits;
    pa.seg = nullptr, pa.status = status;
    if (n_big > 0) {
        pa.sign_mant = sign_mant, pa.codes = codes, pa.tile_base = block_base;
        pa.tb_stride = (int)(big / be), pa.tb_before = 0;
        pa.H = (int)n_big, pa.BH = (int)n_big, pa.seq_tile = 128, pa.D = 128, pa.tile_elems = (int)big;
        pa.n_tiles = n_big, pa.dst = (uint16_t *)dst_bf16;
        pa.db = 0, pa.dh = big, pa.ds = 128;
        int rc = launch_unpack_pipe(pa, st);
        if (rc != ADACODE_OK) return rc;
    }
    const int64_t n_rest = (n_elems - n_main) / be;
    if (n_rest > 0) {
        pa.sign_mant = sign_mant + n_main, pa.codes = codes + n_main * nbits / 8;
        pa.tile_base = block_base + n_main / be;
        pa.tb_stride = 1, pa.tb_before = n_main > 0 ? 1 : 0;
        pa.H = (int)n_rest, pa.BH = (int)n_rest, pa.seq_tile = be / 32, pa.D = 32, pa.tile_elems = be;
        pa.n_tiles = n_rest, pa.dst = (uint16_t *)dst_bf16 + n_main;
        pa.db = 0, pa.dh = be, pa.ds = 32;
        int rc = launch_unpack_pipe(pa, st);
        if (rc != ADACODE_OK) return rc;
    }
    return ADACODE_OK;
}

int adacode_unpack_jobs(const adacode_unpack_job *jobs, int n_jobs, int B, int H, int seq_tile, int D,
                        int32_t *status, void *stream) {
    if (n_jobs < 0 || n_jobs > kMaxJobs || (n_jobs > 0 && !jobs)) return ADACODE_ERR_INVALID_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const bool pipe = pipeline_enabled() && pipeline_shape_ok(seq_tile, D);
    UnpackJobsArgs ja;
    memset(&ja, 0, sizeof(ja));
    int n = 0;
    long long tile0 = 0;
    for (int j = 0; j < n_jobs; ++j) {
        const adacode_unpack_job &jb = jobs[j];
        if (jb.n_segments < 0) return ADACODE_ERR_INVALID_ARG;
        const int64_t n_tiles = (int64_t)B * H * jb.n_segments;
        if (n_tiles == 0) continue;
        int rc = check_unpack_common(B, H, seq_tile, D, jb.dst_bf16, jb.dstride_b, jb.dstride_h, jb.dstride_s, status);
        if (rc != ADACODE_OK) return rc;
        if (!jb.segments_dev) return ADACODE_ERR_INVALID_ARG;
        if (!pipe) {
            rc = adacode_unpack_segments(jb.segments_dev, jb.n_segments, B, H, seq_tile, D, jb.dst_bf16, jb.dstride_b,
                                         jb.dstride_h, jb.dstride_s, status, stream);
            if (rc != ADACODE_OK) return rc;
            continue;
        }
        UnpackPipeArgs &pa = ja.job[n];
        pa.seg = jb.segments_dev;
        pa.H = H, pa.BH = B * H, pa.seq_tile = seq_tile, pa.D = D, pa.tile_elems = seq_tile * D;
        pa.n_tiles = n_tiles, pa.dst = (uint16_t *)jb.dst_bf16;
        pa.db = jb.dstride_b, pa.dh = jb.dstride_h, pa.ds = jb.dstride_s, pa.status = status;
        ja.tile0[n] = tile0;
        tile0 += n_tiles;
        ++n;
    }
    if (!pipe || n == 0) return ADACODE_OK;
    ja.tile0[n] = tile0;
    ja.n_jobs = n;
    return launch_unpack_pipe(ja, st);
}

int adacode_hist_bf16(const void *src_bf16, int64_t stride_b, int64_t stride_h, int64_t stride_s, int B, int H, int S,
                      int D, int32_t *hist256, void *stream) {
    if (B < 0 || H < 0 || S < 0 || D <= 0 || D % 8 != 0 || !hist256) return ADACODE_ERR_INVALID_ARG;
    const int64_t n_rows = (int64_t)B * H * S;
    if (n_rows == 0) return ADACODE_OK;
    if (!src_bf16 || ((uintptr_t)src_bf16 & 15) != 0 || ((stride_b | stride_h | stride_s) & 7))
        return ADACODE_ERR_INVALID_ARG;
    const int64_t n_vec = n_rows * (D / 8);
    int64_t blocks = (n_vec + kThreads * 4 - 1) / (kThreads * 4);
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    k_hist<<<(int)blocks, kThreads, 0, (cudaStream_t)stream>>>((const uint16_t *)src_bf16, stride_b, stride_h,
                                                              stride_s, H, S, D, n_rows, hist256);
    ADACODE_CUDA_TRY(cudaGetLastError());
    return ADACODE_OK;
}

int adacode_choose_params(const int32_t *hist256_dev, int n_hists, int32_t *right_nbits_dev, void *stream) {
    if (n_hists < 0 || (n_hists > 0 && (!hist256_dev || !right_nbits_dev))) return ADACODE_ERR_INVALID_ARG;
    if (n_hists == 0) return ADACODE_OK;
    const int warps_per_block = 4;
    k_choose_params<<<(n_hists + warps_per_block - 1) / warps_per_block, warps_per_block * 32, 0,
                      (cudaStream_t)stream>>>(hist256_dev, n_hists, right_nbits_dev);
    ADACODE_CUDA_TRY(cudaGetLastError());
    return ADACODE_OK;
}

int adacode_choose_params_host(const int64_t *hist256, int *right, int *nbits) {
    return choose_host(hist256, 2, 4, true, right, nbits);
}

int adacode_calibrate_host(const int64_t *hist256, int *right, int *nbits) {
    return choose_host(hist256, 1, 8, false, right, nbits);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// pack without a caller-provided scratch
// ---------------------------------------------------------------------------------------

// Library-owned pack scratch.  In host code this name is only a handle for the runtime's symbol
// lookup, not a device address: the address comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_static_pack_scratch[ADACODE_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void *g_static_scratch_addr[kMaxDevices] = {nullptr};
}  // namespace

extern "C" int adacode_pack_tiles_static(const void *src_bf16, int64_t stride_b, int64_t stride_h, int64_t stride_s,
                                         int B, int H, int n_blocks, int seq_tile, int D, int right, int nbits,
                                         uint8_t *sign_mant, uint8_t *codes, uint8_t *escapes,
                                         int64_t escapes_capacity, int32_t *tile_base, int64_t *seg_escape_offsets,
                                         int32_t *hist256, int32_t *status, void *stream) {
    if (B < 0 || H < 0 || n_blocks < 0 || seq_tile <= 0 || D <= 0) return ADACODE_ERR_INVALID_ARG;
    const int64_t n_tiles = (int64_t)B * H * n_blocks;
    const int64_t tile_elems = (int64_t)seq_tile * D;
    if (n_tiles > 0 && adacode_pack_workspace_bytes(n_tiles, tile_elems) > (size_t)ADACODE_STATIC_SCRATCH_BYTES)
        return ADACODE_ERR_WORKSPACE;   // larger than the built-in scratch: nothing was launched
    int dev = 0;
    ADACODE_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return ADACODE_ERR_INVALID_ARG;
    if (g_static_scratch_addr[dev] == nullptr) {
        // first call on this device (it is the current one): resolve the device address of the array
        void *addr = nullptr;
        ADACODE_CUDA_TRY(cudaGetSymbolAddress(&addr, g_static_pack_scratch));
        if (addr == nullptr) return ADACODE_ERR_CUDA;
        g_static_scratch_addr[dev] = addr;
    }
    void *scratch = g_static_scratch_addr[dev];
    // the completion counter at the head of the scratch must be zero when the kernel starts;
    // whatever an earlier (possibly failed) call left there is cleared in stream order
    ADACODE_CUDA_TRY(cudaMemsetAsync(scratch, 0, 256, (cudaStream_t)stream));
    return adacode_pack_tiles(src_bf16, stride_b, stride_h, stride_s, B, H, n_blocks, seq_tile, D, right, nbits,
                              sign_mant, codes, escapes, escapes_capacity, tile_base, seg_escape_offsets, hist256,
                              scratch, (size_t)ADACODE_STATIC_SCRATCH_BYTES, status, stream);
}
