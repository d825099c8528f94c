// Pipelined pack / unpack kernels: tiles are staged through shared memory with asynchronous
// bulk copies (the untiled form of TMA) so that the loads of the next units are in flight
// while the current unit is processed, and results leave through shared memory with bulk
// stores.  Included by adacode_kernels.cu inside its anonymous namespace.
//
// One CTA = W consumer warps + 1 producer warp, persistent over tiles.  A "unit" is a run of
// whole token rows of one tile, at most W x 1024 elements.  Two geometries are built: the wide one
// (16 warps, units of a whole 128 x 128 tile, 2 CTAs per SM) for the pack kernel and the fused
// attention kernel, the narrow one (8 warps, units of 8192 elements, 4 CTAs per SM) for the unpack
// kernel, which measured 5-8 % faster with four smaller pipelines per SM than with two large ones.
// The pack kernel measured 7 % slower that way (twice the escape slots and unit counts to
// compact) and takes the narrow geometry only for tiles of at most 8192 elements, which would
// leave half the threads of a wide unit idle.
//   producer warp : waits for a free stage, issues the unit's bulk loads (sign/mantissa and
//                   code planes, or source rows) against the stage's "full" mbarrier, and
//                   stages the tile's escape bytes with plain loads
//   consumer warps: wait on "full", work out of shared memory, signal "empty", and hand the
//                   finished unit to a bulk store
// A unit leaves through ONE bulk store per plane: the copy engine has a sizeable cost per
// operation, and a variant in which every consumer warp stored its own 2 KB slice (no CTA-wide
// barrier inside a unit) ran 40 % slower than this one.
// Every mbarrier wait is bounded: after kMaxPolls failed polls the waiter records
// ADACODE_STATUS_TIMEOUT in the status word and carries on (the result is then wrong but the
// kernel still reaches every barrier and terminates).
#pragma once

constexpr int kPCPT = 2;                                   // 16-element chunks per consumer thread and unit

template <int W, int CTAS>
struct PipeGeom {
    static constexpr int kWarps = W;                        // consumer warps
    static constexpr int kConsumers = W * 32;
    static constexpr int kThreads = kConsumers + 32;        // + the producer warp
    static constexpr int kUnit = kConsumers * kPCPT * 16;   // elements per unit
    static constexpr int kCtasPerSm = CTAS;
    static constexpr int kEscStage = kUnit / 2;             // bytes of a tile's escape stream staged with a unit
};
using WideGeom = PipeGeom<16, 2>;
using NarrowGeom = PipeGeom<8, 4>;

// the wide geometry under the names the pack kernel and the attention kernel use
constexpr int kPWarps = WideGeom::kWarps;
constexpr int kConsumerThreads = WideGeom::kConsumers;
constexpr int kPipeThreads = WideGeom::kThreads;
constexpr int kUnitElems = WideGeom::kUnit;
constexpr int kStages = 2;
constexpr uint32_t kMaxPolls = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; on expiry flags the status word and returns anyway (false: the barrier did not
// complete).  Once any wait of the launch has timed out, the others stop waiting as well (they look
// at the status word now and then), so that a broken launch ends in about the time of one expired
// wait.  A consumer whose wait failed keeps computing (it must reach every barrier) but stores
// nothing to global memory any more: it may be looking at a half-written unit description.
__device__ __forceinline__ bool launch_timed_out(const int32_t *status) {
    return (*reinterpret_cast<const volatile int32_t *>(status) & ADACODE_STATUS_TIMEOUT) != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int32_t *status,
                                          uint32_t limit = kMaxPolls) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 4095u) == 4095u && launch_timed_out(status)) return false;
    }
    atomicOr(status, ADACODE_STATUS_TIMEOUT);
    return false;
}
// global -> shared bulk copy, completion counted in bytes on `bar`; 16-byte aligned, size % 16 == 0
__device__ __forceinline__ void bulk_load(void *sdst, const void *gsrc, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(sdst)),
                 "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// shared -> global bulk copy, tracked by the issuing thread's bulk group
__device__ __forceinline__ void bulk_store(void *gdst, const void *ssrc, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(ssrc)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// makes shared-memory writes of this thread visible to the async proxy (bulk stores)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
template <int THREADS = kConsumerThreads>
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory"); }

// Inclusive warp scan of kPCPT per-lane counters walked in (k, lane) order (counters <= 16 each, so
// they travel as 16-bit fields).  incl[k] = inclusive rank of (k, lane) within the warp's
// kPCPT x 32 chunks; returns the warp total.
__device__ __forceinline__ int warp_scan_counts(const int (&cnt)[kPCPT], int (&incl)[kPCPT]) {
    static_assert(kPCPT == 2 || kPCPT == 4, "two or four chunks per thread");
    const int lane = threadIdx.x & 31;
    uint32_t a = (uint32_t)cnt[0] | ((uint32_t)cnt[1] << 16);
    uint32_t b = 0;
    if (kPCPT == 4) b = (uint32_t)cnt[kPCPT - 2] | ((uint32_t)cnt[kPCPT - 1] << 16);
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t ua = __shfl_up_sync(kFull, a, d);
        uint32_t ub = 0;
        if (kPCPT == 4) ub = __shfl_up_sync(kFull, b, d);
        if (lane >= d) {
            a += ua;
            b += ub;
        }
    }
    const uint32_t ta = __shfl_sync(kFull, a, 31);
    const int t0 = ta & 0xFFFF, t1 = ta >> 16;
    incl[0] = (int)(a & 0xFFFF);
    incl[1] = (int)(a >> 16) + t0;
    int total = t0 + t1;
    if (kPCPT == 4) {
        const uint32_t tb = __shfl_sync(kFull, b, 31);
        incl[kPCPT - 2] = (int)(b & 0xFFFF) + total;
        incl[kPCPT - 1] = (int)(b >> 16) + total + (int)(tb & 0xFFFF);
        total += (int)(tb & 0xFFFF) + (int)(tb >> 16);
    }
    return total;
}

// Exclusive prefix of this warp and the total over all consumer warps, from the per-warp totals
// in shared memory: lane i reads warp i's total, one warp scan, two shuffles.
template <int W = kPWarps>
__device__ __forceinline__ void cross_warp_prefix(const int *warp_tot, int &prefix, int &total) {
    static_assert(W <= 32, "one lane per consumer warp");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int x = lane < W ? warp_tot[lane] : 0;
#pragma unroll
    for (int d = 1; d < W; d <<= 1) {
        const int u = __shfl_up_sync(kFull, x, d);
        if (lane >= d) x += u;
    }
    total = __shfl_sync(kFull, x, W - 1);
    const int incl = __shfl_sync(kFull, x, warp);
    const int own = __shfl_sync(kFull, lane < W ? warp_tot[lane] : 0, warp);
    prefix = incl - own;
}

// Rows of one tile handled per unit: whole rows, a multiple of 8 (so that code bytes per unit are a
// multiple of 16), at most UNIT elements (D <= UNIT / 8).
template <int UNIT = kUnitElems>
__host__ __device__ inline int unit_rows_for(int seq_tile, int D) {
    int r = (UNIT / D) & ~7;
    if (r < 8) r = 8;
    return r < seq_tile ? r : seq_tile;
}

// ---------------------------------------------------------------------------------------
// unpack
// ---------------------------------------------------------------------------------------

constexpr int kEscStage = WideGeom::kEscStage;

struct UnitMeta {
    uint16_t *dst;            // first element of the unit in the destination
    const uint8_t *esc;       // the segment's escape stream
    long long esc_len;
    long long esc_tile_start; // index in esc of the tile's first escape
    int esc_staged;           // escapes of the tile present in shared memory (from index 0 of the tile)
    int esc_shift;            // offset of escape 0 inside the staged bytes
    int elems;
    int left;
    int nbits;
    int first_unit_of_tile;
    long long ds;             // destination row stride in elements
};

// bulk copies need 16-byte aligned shared addresses: every buffer starts on a 128-byte boundary
template <class G>
struct alignas(128) UnpackStageT {
    alignas(128) uint8_t sm[G::kUnit];
    alignas(128) uint8_t codes[G::kUnit / 2];
    alignas(128) uint8_t esc[G::kEscStage + 16];
    alignas(16) UnitMeta meta;
};

template <class G>
struct alignas(128) UnpackSmemT {
    UnpackStageT<G> stage[kStages];
    alignas(128) uint16_t out[G::kUnit];
    alignas(16) uint32_t lut[1024];   // decode table of the current (left, nbits)
    // Unit descriptions live in a ring of their own, twice as deep as the stages: a consumer reads
    // the destination of unit i after it has released stage i % kStages, and the producer writes
    // the description of unit i + 2 * kStages only after every consumer has released unit
    // i + kStages, i.e. after it is done with unit i altogether.  So nobody has to keep a
    // description in registers through a unit.
    alignas(16) UnitMeta meta_ring[2 * kStages];
    alignas(8) uint64_t full[kStages];
    alignas(8) uint64_t empty[kStages];
    int warp_tot[G::kWarps];
};
using UnpackStage = UnpackStageT<WideGeom>;
static_assert(sizeof(UnpackStageT<WideGeom>) % 128 == 0 && sizeof(UnpackStageT<NarrowGeom>) % 128 == 0,
              "stage buffers must stay 128-byte aligned");

struct UnpackPipeArgs {
    // uniform form (seg == nullptr): planes as adacode_pack_tiles wrote them
    const uint8_t *sign_mant;
    const uint8_t *codes;
    const uint8_t *escapes;
    long long escapes_len;
    const int32_t *tile_base;
    const int64_t *seg_off;
    int left, nbits;
    int tb_stride;            // tile t's inclusive base is tile_base[(t + 1) * tb_stride - 1] (1: one entry per tile)
    int tb_before;            // tile_base[-1] exists and holds the escapes before tile 0
    // table form
    const adacode_segment *seg;
    // common
    int H, BH, seq_tile, D, tile_elems;
    long long n_tiles;
    uint16_t *dst;
    long long db, dh, ds;
    int32_t *status;
};

// Everything the producer needs to know about tile `tile`.
struct TileSrc {
    const uint8_t *sm, *codes, *esc;
    long long esc_len, esc_start;
    int esc_cnt, left, nbits;
    uint16_t *dst;
    long long ds;
};

__device__ __forceinline__ TileSrc resolve_tile(const UnpackPipeArgs &a, long long tile) {
    TileSrc t;
    const long long blk = tile / a.BH;
    const int bh = (int)(tile - blk * a.BH);
    const int b = bh / a.H, h = bh - b * a.H;
    uint16_t *base = a.dst + (long long)b * a.db + (long long)h * a.dh;
    t.ds = a.ds;
    if (a.seg) {
        const adacode_segment sg = a.seg[blk];
        t.nbits = sg.nbits, t.left = sg.left;
        t.sm = sg.sign_mant + (long long)bh * a.tile_elems;
        t.codes = sg.codes + (long long)bh * (a.tile_elems * sg.nbits / 8);
        t.esc = sg.escapes, t.esc_len = sg.escapes_len;
        const int prev = bh > 0 ? sg.tile_base[bh - 1] : 0;
        t.esc_start = prev;
        t.esc_cnt = sg.tile_base[bh] - prev;
        t.dst = base + sg.dst_seq_offset * a.ds;
    } else {
        t.nbits = a.nbits, t.left = a.left;
        t.sm = a.sign_mant + tile * a.tile_elems;
        t.codes = a.codes + tile * (a.tile_elems * a.nbits / 8);
        t.esc = a.escapes, t.esc_len = a.escapes_len;
        const long long seg_start = a.seg_off ? a.seg_off[blk] : 0;
        const long long ts = a.tb_stride > 1 ? a.tb_stride : 1;
        const int prev = (bh > 0 || a.tb_before) ? a.tile_base[tile * ts - 1] : 0;
        t.esc_start = seg_start + prev;
        t.esc_cnt = a.tile_base[tile * ts + ts - 1] - prev;
        t.dst = base + blk * a.seq_tile * a.ds;
    }
    return t;
}

__device__ __forceinline__ long long shfl_ll(long long v, int src) {
    const int lo = __shfl_sync(kFull, (int)(v & 0xFFFFFFFFll), src);
    const int hi = __shfl_sync(kFull, (int)(v >> 32), src);
    return ((long long)hi << 32) | (unsigned int)lo;
}
template <typename T>
__device__ __forceinline__ T *shfl_ptr(T *p, int src) {
    return reinterpret_cast<T *>(shfl_ll((long long)(uintptr_t)p, src));
}
// Lane `src`'s tile description, in every lane of the warp.
__device__ __forceinline__ TileSrc shfl_tile(const TileSrc &m, int src) {
    TileSrc t;
    t.sm = shfl_ptr(m.sm, src), t.codes = shfl_ptr(m.codes, src), t.esc = shfl_ptr(m.esc, src);
    t.esc_len = shfl_ll(m.esc_len, src), t.esc_start = shfl_ll(m.esc_start, src);
    t.esc_cnt = __shfl_sync(kFull, m.esc_cnt, src);
    t.left = __shfl_sync(kFull, m.left, src), t.nbits = __shfl_sync(kFull, m.nbits, src);
    t.dst = shfl_ptr(m.dst, src);
    t.ds = shfl_ll(m.ds, src);
    return t;
}

// The part of a tile's escape stream that is staged in shared memory with each of its units.
// The window [a0, a0 + win) of whole 16-byte granules is fetched with one bulk copy.  It may
// begin up to 15 bytes before the tile's first escape (same granule, ignored), but never reaches
// past the last whole granule of the stream: what lies in the stream's final partial granule
// (`tail` bytes) is fetched with plain loads.
struct EscWindow {
    const uint8_t *a0;
    int win, tail, staged, shift;
};

template <int ESC_STAGE = kEscStage>
__device__ __forceinline__ EscWindow esc_window(const TileSrc &t) {
    EscWindow w;
    // stage no more than the stream really holds, so that a short stream is reported as such
    long long avail = t.esc_len - t.esc_start;
    if (avail > t.esc_cnt) avail = t.esc_cnt;
    if (avail > ESC_STAGE) avail = ESC_STAGE;
    w.staged = avail > 0 ? (int)avail : 0;
    const uint8_t *ea = t.esc + t.esc_start;
    w.shift = (int)((uintptr_t)ea & 15);
    w.a0 = ea - w.shift;
    w.win = (w.shift + w.staged + 15) & ~15;
    w.tail = 0;
    const uintptr_t stream_end = (uintptr_t)(t.esc + t.esc_len);
    if (w.staged > 0 && (uintptr_t)w.a0 + (uintptr_t)w.win > stream_end) {
        w.win -= 16;
        w.tail = (int)(stream_end & 15);
    }
    if (w.staged == 0) w.win = 0;
    return w;
}

// Producer warp, stage known to be free: describe the unit (rows [row0, row0 + rows) of tile t) in
// `m` and start its bulk copies against `full_bar`.
template <class Stage>
__device__ __forceinline__ void issue_unit(Stage &st, UnitMeta &m, uint64_t *full_bar, const TileSrc &t,
                                           const EscWindow &w, int row0, int rows, int D, uint16_t *dst,
                                           bool first_unit, int32_t *status, bool withhold = false) {
    const int lane = threadIdx.x & 31;
    if (w.tail > 0) {
        if (lane < w.tail) st.esc[w.win + lane] = w.a0[w.win + lane];
        __syncwarp();
    }
    if (lane == 0) {
        const int elems = rows * D;
        const uint8_t *src_sm = t.sm + (long long)row0 * D;
        const uint8_t *src_cd = t.codes + (long long)row0 * D * t.nbits / 8;
        m.dst = dst;
        m.esc = t.esc, m.esc_len = t.esc_len, m.esc_tile_start = t.esc_start;
        m.esc_staged = w.staged, m.esc_shift = w.shift;
        m.elems = elems, m.left = t.left, m.nbits = t.nbits;
        m.first_unit_of_tile = first_unit;
        m.ds = t.ds;
        const uint32_t cbytes = (uint32_t)elems * t.nbits / 8;
        if (withhold) {
            // testing aid: an empty unit whose "loaded" signal never comes; the consumers' bounded
            // wait runs out, they flag ADACODE_STATUS_TIMEOUT and carry on with nothing to do
            m.elems = 0;
            m.nbits = 1;
        } else if ((((uintptr_t)src_sm | (uintptr_t)src_cd | (uintptr_t)dst) & 15) != 0 || (cbytes & 15) != 0 || t.nbits < 1 ||
            t.nbits > 4) {
            // never start a misaligned bulk copy: flag it and hand over an empty unit
            atomicOr(status, ADACODE_STATUS_MISALIGNED);
            m.elems = 0;
            m.nbits = 1;
            mbar_arrive_expect_tx(full_bar, 0);
        } else {
            mbar_arrive_expect_tx(full_bar, (uint32_t)elems + cbytes + (uint32_t)w.win);
            bulk_load(st.sm, src_sm, (uint32_t)elems, full_bar);
            bulk_load(st.codes, src_cd, cbytes, full_bar);
            if (w.win > 0) bulk_load(st.esc, w.a0, (uint32_t)w.win, full_bar);
        }
    }
}

// Register phase of a unit, shared by the unpack kernel and the fused attention kernel: every
// consumer thread decodes its kPCPT chunks of the staged planes into registers (exponent fields
// from the table, 0 where the code is 0; sign and mantissa merged in) and notes where the
// escapes are (zm: one bit per code-0 slot of each group word; zc: their number per chunk).
template <int N, class Stage>
__device__ __forceinline__ void decode_chunks(const Stage &st, const uint32_t *lut, int chunks,
                                              uint4 (&o)[kPCPT][2], uint32_t (&zm)[kPCPT][2], int (&zc)[kPCPT]) {
    constexpr int CB = 2 * N;   // code bytes per 16-element chunk
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < kPCPT; ++k) {
        const int c = warp * (kPCPT * 32) + k * 32 + lane;
        uint32_t g[2] = {0u, 0u};
        uint4 sv = make_uint4(0, 0, 0, 0);
        const bool valid = c < chunks;
        if (valid) {
            sv = *reinterpret_cast<const uint4 *>(st.sm + c * 16);
            load_chunk_codes<N, 16>(st.codes + c * CB, g);
        }
        const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
        zc[k] = 0;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            zm[k][q] = valid ? zero_slots<N>(g[q]) : 0u;
            zc[k] += __popc(zm[k][q]);
            uint32_t ew[4];
            decode_group<N>(lut, g[q], ew);
            const uint32_t s0 = sw[2 * q], s1 = sw[2 * q + 1];
            // sign and mantissa: each byte doubled into its 16-bit lane, then masked into place
            o[k][q].x = ew[0] | (__byte_perm(s0, 0u, 0x1100) & 0x807F807Fu);
            o[k][q].y = ew[1] | (__byte_perm(s0, 0u, 0x3322) & 0x807F807Fu);
            o[k][q].z = ew[2] | (__byte_perm(s1, 0u, 0x1100) & 0x807F807Fu);
            o[k][q].w = ew[3] | (__byte_perm(s1, 0u, 0x3322) & 0x807F807Fu);
        }
    }
}

template <int N, class G>
__device__ __forceinline__ void unpack_unit(UnpackSmemT<G> &s, const UnpackStageT<G> &st, const UnitMeta &meta,
                                            uint64_t *empty_bar, int &consumed, int D, int32_t *status, bool broken) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // only what the common path needs is read from the unit's description up front; the fields of
    // the rare global-memory escape path and the destination are read where they are used
    const int esc_staged = meta.esc_staged, esc_shift = meta.esc_shift;
    if (meta.first_unit_of_tile) consumed = 0;
    const int chunks = meta.elems >> 4;

    uint4 o[kPCPT][2];
    uint32_t zm[kPCPT][2];
    int zc[kPCPT];
    decode_chunks<N>(st, s.lut, chunks, o, zm, zc);
    int incl[kPCPT];
    const int wtot = warp_scan_counts(zc, incl);
    if (lane == 0) s.warp_tot[warp] = wtot;
    bulk_wait_read();          // the previous unit's store has finished reading s.out
    consumer_sync<G::kConsumers>();
    int wprefix, unit_tot;
    cross_warp_prefix<G::kWarps>(s.warp_tot, wprefix, unit_tot);
    static_assert(kPCPT == 2, "the escape loop below walks the two chunks of a thread together");
    const int c0 = warp * (kPCPT * 32) + lane;
#pragma unroll
    for (int k = 0; k < kPCPT; ++k) {
        const int c = c0 + k * 32;
        if (c < chunks) {
            uint16_t *ow = s.out + c * 16;
            reinterpret_cast<uint4 *>(ow)[0] = o[k][0];
            reinterpret_cast<uint4 *>(ow)[1] = o[k][1];
        }
    }
    if (zc[0] + zc[1] != 0) {
        // ranks inside the tile of the first escape of either chunk
        const int r0 = consumed + wprefix + incl[0] - zc[0], r1 = consumed + wprefix + incl[1] - zc[1];
        const bool staged = (zc[0] == 0 || r0 + zc[0] <= esc_staged) && (zc[1] == 0 || r1 + zc[1] <= esc_staged);
        if (staged) {
            // One loop over the escapes of both chunks (four groups): a warp iterates as often as its
            // busiest lane has escapes, and per-lane totals over 32 elements vary much less than
            // per-group counts over 8, so this takes about half the iterations of four separate loops.
            // mask: chunk 0 elements 0..15, then chunk 1 elements 0..15, from the most significant bit.
            uint32_t todo = (compress_slots<N>(zm[0][0]) << 24) | (compress_slots<N>(zm[0][1]) << 16) |
                            (compress_slots<N>(zm[1][0]) << 8) | compress_slots<N>(zm[1][1]);
            // The exponent field in s.out is zero at escaped positions (code 0 decodes to 0), so the
            // escape byte is OR-ed in with a shared-memory reduction: no read-modify-write round trip.
            const uint8_t *ep = st.esc + esc_shift + r0;
            const int skip = r1 - r0 - zc[0];             // from chunk 0's escapes to chunk 1's
            uint32_t *ow32 = reinterpret_cast<uint32_t *>(s.out + c0 * 16);
            int n = 0;
            while (todo) {
                const int i = __clz(todo);
                todo &= ~(0x80000000u >> i);
                const uint32_t e = ep[n + (i >> 4) * skip];
                ++n;
                // chunk 1 lies 32 chunks = 256 words further on; (i >> 1) & 7 is the word inside the chunk
                atomicOr(ow32 + (((i >> 4) << 8) | ((i >> 1) & 7)), e << (7 + 16 * (i & 1)));
            }
        } else {
            // beyond the staged window (or beyond the stream): fetch from global memory
            const uint8_t *g_esc = meta.esc;
            const long long g_len = meta.esc_len, g_start = meta.esc_tile_start;
#pragma unroll 1
            for (int k = 0; k < kPCPT; ++k) {
                uint16_t *ow = s.out + (c0 + k * 32) * 16;
                int r = k == 0 ? r0 : r1;
#pragma unroll 1
                for (int q = 0; q < 2; ++q) {
                    // (selects, not zm[k][q]: a run-time index would move the array to local memory)
                    uint32_t z = k == 0 ? (q == 0 ? zm[0][0] : zm[0][1]) : (q == 0 ? zm[1][0] : zm[1][1]);
                    while (z) {
                        const int pos = 31 - __clz(z);
                        z ^= 1u << pos;
                        uint32_t e = 0;
                        if (r < esc_staged) e = st.esc[esc_shift + r];
                        else if (g_start + r < g_len) e = g_esc[g_start + r];
                        else atomicOr(status, ADACODE_STATUS_ESCAPE_UNDERRUN);
                        ++r;
                        uint16_t *pw = ow + (q * 8 + 7 - pos / N);
                        *pw = (uint16_t)((*pw & 0x807Fu) | (e << 7));
                    }
                }
            }
        }
    }
    consumed += unit_tot;
    mbar_arrive(empty_bar);    // this thread no longer reads the stage
    fence_async_smem();
    consumer_sync<G::kConsumers>();
    const long long ds = meta.ds;
    if (broken) {
        // (nothing is stored)
    } else if (ds == D) {
        if (tid == 0 && meta.elems > 0) {
            bulk_store(meta.dst, s.out, (uint32_t)meta.elems * 2u);
            bulk_commit();
        }
    } else {
        const int rows = meta.elems / D;
        uint16_t *const dst = meta.dst;
        for (int r = tid; r < rows; r += G::kConsumers) bulk_store(dst + (long long)r * ds, s.out + r * D, (uint32_t)D * 2u);
        bulk_commit();
    }
}

// Consumer warp: wait (bounded) until unit `it` is loaded; false if the wait gave up.
template <class G>
__device__ __forceinline__ bool wait_loaded(UnpackSmemT<G> &s, uint32_t it, int32_t *status, uint32_t poll_limit) {
    bool loaded = true;
    if ((threadIdx.x & 31) == 0) loaded = mbar_wait(&s.full[it % kStages], (it / kStages) & 1, status, poll_limit);
    loaded = __shfl_sync(kFull, loaded, 0);
    __syncwarp();          // orders the other lanes' reads of the stage after lane 0's wait
    return loaded;
}

// Units it, it + 1, ... as long as they carry code length N and window `left` (the decode table
// in s.lut); returns the first unit that does not, already waited for, or n_units.
template <int N, class G>
__device__ __forceinline__ uint32_t unpack_run(UnpackSmemT<G> &s, uint32_t it, uint32_t n_units, int left, int &consumed,
                                               bool &broken, int D, int32_t *status, uint32_t poll_limit) {
    for (;;) {
        const int stg = it % kStages;
        unpack_unit<N>(s, s.stage[stg], s.meta_ring[it % (2 * kStages)], &s.empty[stg], consumed, D, status, broken);
        if (++it >= n_units) return it;
        broken |= !wait_loaded(s, it, status, poll_limit);
        const UnitMeta &next = s.meta_ring[it % (2 * kStages)];
        if (next.nbits != N || next.left != left) return it;
    }
}

constexpr int kMaxJobs = 8;

// Up to kMaxJobs destinations in one launch; job j owns the tiles [tile0[j], tile0[j + 1]).
struct UnpackJobsArgs {
    UnpackPipeArgs job[kMaxJobs];
    long long tile0[kMaxJobs + 1];
    int n_jobs;
    uint32_t poll_limit;      // bound of every on-chip wait (kMaxPolls unless a test lowered it)
    int withhold_unit;        // testing aid: CTA 0's producer never signals this unit as loaded (-1: off)
};

template <class G>
__global__ void __launch_bounds__(G::kThreads, G::kCtasPerSm) k_unpack_pipe(const __grid_constant__ UnpackJobsArgs ja) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    UnpackSmemT<G> &s = *reinterpret_cast<UnpackSmemT<G> *>(smem_raw);
    const int tid = threadIdx.x;
    const UnpackPipeArgs &a0 = ja.job[0];          // geometry and status word are common to all jobs
    const long long n_tiles = ja.tile0[ja.n_jobs];
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], G::kConsumers);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid < 2 * kStages) {
        // an empty unit: what a consumer sees if it gives up waiting before the first description is written
        UnitMeta &m = s.meta_ring[tid];
        m.dst = nullptr, m.esc = nullptr, m.esc_len = 0, m.esc_tile_start = 0, m.esc_staged = 0, m.esc_shift = 0;
        m.elems = 0, m.left = 0, m.nbits = 1, m.first_unit_of_tile = 1, m.ds = 0;
    }
    __syncthreads();
    // launched as a programmatic dependent of its predecessor in the stream: no global memory is touched above
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int unit_rows = unit_rows_for<G::kUnit>(a0.seq_tile, a0.D);
    const int units_per_tile = (a0.seq_tile + unit_rows - 1) / unit_rows;

    if (tid >= G::kConsumers) {
        // ---------------- producer warp ----------------
        // Tile metadata sits behind two dependent global loads (segment record, then the tile's
        // escape range).  Each lane resolves one of this CTA's next 32 tiles, so those round trips
        // are paid once per 32 tiles and never between "stage free" and "loads issued".
        const int lane = tid & 31;
        uint32_t it = 0;
        const long long my_tiles =
            n_tiles > (long long)blockIdx.x ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        for (long long base = 0; base < my_tiles; base += 32) {
            TileSrc mine = {};
            if (base + lane < my_tiles) {
                const long long tile = blockIdx.x + (base + lane) * (long long)gridDim.x;
                int j = 0;
                while (j + 1 < ja.n_jobs && tile >= ja.tile0[j + 1]) ++j;
                mine = resolve_tile(ja.job[j], tile - ja.tile0[j]);
            }
            const int n_here = (int)(my_tiles - base < 32 ? my_tiles - base : 32);
            for (int j = 0; j < n_here; ++j) {
                const TileSrc t = shfl_tile(mine, j);
                const EscWindow w = esc_window<G::kEscStage>(t);
                for (int u = 0; u < units_per_tile; ++u, ++it) {
                    const int stg = it % kStages;
                    mbar_wait(&s.empty[stg], ((it / kStages) & 1) ^ 1, a0.status, ja.poll_limit);
                    const int row0 = u * unit_rows;
                    const int rows = min(unit_rows, a0.seq_tile - row0);
                    issue_unit(s.stage[stg], s.meta_ring[it % (2 * kStages)], &s.full[stg], t, w, row0, rows, a0.D,
                               t.dst + (long long)row0 * t.ds,
                               u == 0, a0.status, blockIdx.x == 0 && (int)it == ja.withhold_unit);
                }
            }
        }
        // Do not leave while a copy into this CTA's shared memory may still be in flight: after a
        // timed-out launch the consumers can be ahead of the data (a bounded wait, like all others).
        if (launch_timed_out(a0.status))
            for (uint32_t k = it > kStages ? it - kStages : 0; k < it; ++k)
                if (!(blockIdx.x == 0 && (int)k == ja.withhold_unit))
                    mbar_wait(&s.full[k % kStages], (k / kStages) & 1, a0.status, ja.poll_limit);
        return;
    }

    // ---------------- consumer warps ----------------
    int consumed = 0;
    bool broken = false;                  // a wait of this warp ran out: compute on, store nothing
    int lut_left = 0, lut_nbits = 0;      // what s.lut currently encodes (nbits 0: nothing yet)
    // (the consumers only count units: which tile a unit belongs to is in its description)
    const uint32_t my_units =
        n_tiles > (long long)blockIdx.x
            ? (uint32_t)((n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x) * (uint32_t)units_per_tile
            : 0u;
    // Units of one code length and window are handled by a loop of their own (unpack_run<N>), so
    // that the compiler schedules each code length's loop body by itself; this outer loop only
    // takes over when the table has to change.
    uint32_t it = 0;
    while (it < my_units) {
        broken |= !wait_loaded(s, it, a0.status, ja.poll_limit);      // returns at once if unpack_run waited already
        const UnitMeta &meta = s.meta_ring[it % (2 * kStages)];
        const int nb = meta.nbits, lf = meta.left;
        if (nb != lut_nbits || lf != lut_left) {
            // uniform over the CTA: every consumer read the same description.  The previous unit
            // ended with a consumer barrier, so nobody still reads the old table.
            build_decode_lut(s.lut, nb, lf, G::kConsumers);
            lut_nbits = nb, lut_left = lf;
            consumer_sync<G::kConsumers>();
        }
        switch (nb) {
            case 1: it = unpack_run<1>(s, it, my_units, lf, consumed, broken, a0.D, a0.status, ja.poll_limit); break;
            case 2: it = unpack_run<2>(s, it, my_units, lf, consumed, broken, a0.D, a0.status, ja.poll_limit); break;
            case 3: it = unpack_run<3>(s, it, my_units, lf, consumed, broken, a0.D, a0.status, ja.poll_limit); break;
            default: it = unpack_run<4>(s, it, my_units, lf, consumed, broken, a0.D, a0.status, ja.poll_limit); break;
        }
    }
    bulk_wait_all();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

#ifndef ADACODE_PIPELINE_UNPACK_ONLY
// ---------------------------------------------------------------------------------------
// pack
// ---------------------------------------------------------------------------------------

// In-window histogram over several group words at once.  Bit i of a code lands on the least
// significant bit of its N-bit slot, so N groups (4 for N <= 2) can be overlaid on one 32-bit
// word: plane[i] then holds bit i of up to 32 codes.
//
// What is counted is not "how many codes equal v" (one three-input AND with complements, a mask
// and a population count per value) but, for every non-empty proper subset m of the N code bits,
// "how many codes have all bits of m set" (f(m): one AND of the planes named by m, no AND at all
// for single bits).  Together with the number of elements f(0) and the number of escapes x(0),
// which the kernel knows anyway, the per-value counts follow at flush time by inverting the
// superset sums: f(full) = (-1)^N (x(0) - sum_{m != full} (-1)^|m| f(m)), then
// x(c) = sum_{m >= c} (-1)^(|m|-|c|) f(m).  For N = 3 that is 6 population counts and 3 ANDs per
// 24 elements instead of 7 and 14; for N = 1 nothing at all.
template <int N>
struct GroupsPerWord { static constexpr int v = (N == 3) ? 3 : 4; };

template <int N>
__device__ __forceinline__ uint32_t overlay_shift(int j) {
    if (N >= 3) return (uint32_t)j;                           // sub-slot offsets 0..N-1
    if (N == 2) return (uint32_t)((j & 1) + 16 * (j >> 1));   // 16-bit halves, two sub-slot offsets
    return (uint32_t)(8 * j);                                 // N == 1: one byte per group
}

// Counters live in registers, two 16-bit fields per register: field 0 counts elements, field m
// (0 < m < 2^N - 1) the codes with all bits of m set, field 2^N - 1 the escapes.  A thread adds at
// most 32 to a field per unit, so the fields are flushed every 1024 units at the latest.
template <int N>
struct HistRegs { static constexpr int v = (1 << N) / 2 > 0 ? (1 << N) / 2 : 1; };

template <int N>
__device__ __forceinline__ void bump_field(uint32_t (&cnt2)[HistRegs<N>::v], int field, uint32_t by) {
    cnt2[field >> 1] = by * ((field & 1) ? 65536u : 1u) + cnt2[field >> 1];
}

template <int N, int NG>
__device__ __forceinline__ void count_codes_overlaid(const uint32_t (&g)[NG], uint32_t (&cnt2)[HistRegs<N>::v]) {
    constexpr int GPW = GroupsPerWord<N>::v;
    constexpr int FULL = (1 << N) - 1;
    constexpr uint32_t M = SlotLsb<N>::v;
#pragma unroll
    for (int base = 0; base < NG; base += GPW) {
        uint32_t plane[N];
#pragma unroll
        for (int i = 0; i < N; ++i) plane[i] = 0;
#pragma unroll
        for (int j = 0; j < GPW; ++j) {
            if (base + j < NG) {
                const uint32_t sh = overlay_shift<N>(j);
#pragma unroll
                for (int i = 0; i < N; ++i) plane[i] = ((g[base + j] >> i) & M) * (1u << sh) + plane[i];
            }
        }
#pragma unroll
        for (int m = 1; m < FULL; ++m) {
            uint32_t all = 0xFFFFFFFFu;
#pragma unroll
            for (int i = 0; i < N; ++i)
                if ((m >> i) & 1) all &= plane[i];
            bump_field<N>(cnt2, m, (uint32_t)__popc(all));
        }
    }
}

struct PackUnitMeta {
    uint8_t *sm_dst;       // sign/mantissa bytes of the unit
    uint8_t *code_dst;     // code bytes of the unit
    uint8_t *esc_dst;      // the unit's escape slot in the scratch
    int32_t *unit_count;   // where the unit's escape count goes
    int32_t *tile_count;   // where the tile's escape count goes (written with the last unit)
    int elems;
    int first_unit_of_tile;
    int last_unit_of_tile;
    int job;               // index into PackPipeArgs::job
};

template <class G>
struct alignas(128) PackStageT {
    alignas(128) uint16_t in[G::kUnit];
};

template <class G>
struct alignas(128) PackSmemT {
    PackStageT<G> stage[kStages];
    alignas(128) uint8_t sm[G::kUnit];
    alignas(128) uint8_t codes[G::kUnit / 2];
    alignas(128) uint8_t esc[G::kUnit];      // worst case: every element of a unit escapes
    alignas(16) uint8_t lut[256];      // exponent -> code (0 = outside the window)
    alignas(16) PackUnitMeta meta_ring[2 * kStages];   // unit descriptions (see UnpackSmemT::meta_ring)
    alignas(8) uint64_t full[kStages];
    alignas(8) uint64_t empty[kStages];
    int warp_tot[G::kWarps];
    int hist[256];
    int is_last;
    long long carry;
    long long job_off[kMaxJobs];
    int scan[G::kWarps];
};
static_assert(sizeof(PackStageT<WideGeom>) % 128 == 0 && sizeof(PackStageT<NarrowGeom>) % 128 == 0,
              "stage buffers must stay 128-byte aligned");

// One tensor of a pack launch.  All jobs of a launch share B, H, seq_tile, D and the code length;
// job j owns the global tiles [tile0, tile0 + BH * n_blocks) and the global blocks [blk0, blk0 + n_blocks).
struct PackJob {
    const uint16_t *src;
    int64_t sb, sh, ss;
    uint8_t *sign_mant, *codes, *escapes;
    int64_t capacity;
    int32_t *tile_base;
    int64_t *seg_off;
    int32_t *hist;           // nullable
    int64_t tile0;
    int blk0, n_blocks, left, pad;
};

struct PackPipeArgs {
    PackJob job[kMaxJobs];
    int n_jobs;
    int H, BH, seq_tile, D, tile_elems;
    int64_t n_tiles;          // over all jobs
    uint8_t *esc_scratch;     // n_tiles * tile_elems bytes, global tile t owns [t * tile_elems, ...)
    int32_t *tile_counts;     // n_tiles
    int32_t *unit_counts;     // n_tiles * units_per_tile
    int64_t *blk_off;         // over all blocks of the launch: escapes before global block i (n_blocks_total + 1)
    unsigned int *done;       // zero on entry, zero on exit
    int unit_rows, units_per_tile;
    int32_t *status;
    uint32_t poll_limit;      // bound of every on-chip wait (kMaxPolls unless a test lowered it)
};

__device__ __forceinline__ int job_of_tile(const PackPipeArgs &pa, int64_t tile) {
    int j = 0;
    while (j + 1 < pa.n_jobs && tile >= pa.job[j + 1].tile0) ++j;
    return j;
}

// Turn per-tile escape counts into per-segment inclusive tile bases and segment offsets (per job).
// Run by the consumer threads of the CTA that finished last, while the rest of the GPU is idle,
// so it is kept short: every thread takes a run of kScanRun consecutive tiles; the counts of the
// next pass (threads x kScanRun tiles) are fetched while the current pass is worked on, so the
// memory round trip of a pass is hidden; one block scan of the run totals gives every tile its
// prefix; and the escape offsets of the blocks that begin inside the pass travel through shared
// memory (`boff`, one entry per block touched by the pass, in the idle staging buffers), not
// through global memory.
constexpr int kScanRun = 8;

template <class G>
__device__ __forceinline__ void scan_tile_counts(const PackPipeArgs &pa, long long *s_carry, int *s_scan,
                                                 long long *s_job_off, long long *boff_raw) {
    // All offsets of a launch fit 32 bits (it has fewer than 2**31 elements), and a thread walks
    // consecutive tiles, so block index, position in the block and job advance by comparison:
    // one division per thread and pass.  (One SM does all of this while the others wait.)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int per_pass = G::kConsumers * kScanRun;
    const int n_tiles = (int)pa.n_tiles, BH = pa.BH;
    int *carry = reinterpret_cast<int *>(s_carry);
    int *job_off = reinterpret_cast<int *>(s_job_off);
    int *boff = reinterpret_cast<int *>(boff_raw);
    if (tid == 0) {
        *carry = 0;
        pa.blk_off[0] = 0;
        boff[0] = 0;
    }
    if (tid < kMaxJobs) job_off[tid] = 0;
    if (tid < pa.n_jobs) pa.job[tid].seg_off[0] = 0;
    int c[kScanRun], nxt[kScanRun];
#pragma unroll
    for (int i = 0; i < kScanRun; ++i) {
        const int t = tid * kScanRun + i;
        c[i] = t < n_tiles ? __ldcg(pa.tile_counts + t) : 0;
    }
    consumer_sync<G::kConsumers>();
    for (int pass = 0; pass < n_tiles; pass += per_pass) {
        const int t0 = pass + tid * kScanRun;
#pragma unroll
        for (int i = 0; i < kScanRun; ++i) {
            const int t = t0 + per_pass + i;
            nxt[i] = t < n_tiles ? __ldcg(pa.tile_counts + t) : 0;
        }
        int run = 0;
#pragma unroll
        for (int i = 0; i < kScanRun; ++i) run += c[i];
        int x = run;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int u = __shfl_up_sync(kFull, x, d);
            if (lane >= d) x += u;
        }
        if (lane == 31) s_scan[warp] = x;
        consumer_sync<G::kConsumers>();
        int wp = 0, tot = 0;
#pragma unroll
        for (int i = 0; i < G::kWarps; ++i) {
            const int v = s_scan[i];
            wp += (i < warp) ? v : 0;
            tot += v;
        }
        const int gb0 = pass / BH;                        // the block the pass begins in; boff[0] is its offset
        const int gb_first = t0 / BH, rem_first = t0 - gb_first * BH;
        int incl = *carry + wp + (x - run);               // escapes before this thread's run
        int inc[kScanRun];
        {
            int gb = gb_first, rem = rem_first;
#pragma unroll
            for (int i = 0; i < kScanRun; ++i) {
                incl += c[i];
                inc[i] = incl;                            // inclusive prefix over the whole launch
                if (++rem == BH) {                        // tile t0 + i ends block gb
                    rem = 0;
                    ++gb;
                    if (t0 + i < n_tiles) {
                        pa.blk_off[gb] = incl;
                        boff[gb - gb0] = incl;
                        for (int j = 1; j < pa.n_jobs; ++j)
                            if (pa.job[j].blk0 == gb) job_off[j] = incl;
                    }
                }
            }
        }
        consumer_sync<G::kConsumers>();                   // the offsets of the blocks of this pass are in boff
        if (t0 < n_tiles) {
            int gb = gb_first, rem = rem_first;
            int j = job_of_tile(pa, t0);
            int j_end = j + 1 < pa.n_jobs ? (int)pa.job[j + 1].tile0 : n_tiles;
            int32_t *tb = pa.job[j].tile_base - pa.job[j].tile0;
            int start = boff[gb - gb0];                   // offset at which block gb begins
#pragma unroll
            for (int i = 0; i < kScanRun; ++i) {
                const int t = t0 + i;
                if (t < n_tiles) {
                    if (t == j_end) {
                        ++j;
                        j_end = j + 1 < pa.n_jobs ? (int)pa.job[j + 1].tile0 : n_tiles;
                        tb = pa.job[j].tile_base - pa.job[j].tile0;
                    }
                    tb[t] = inc[i] - start;
                    if (++rem == BH) {
                        rem = 0;
                        ++gb;
                        pa.job[j].seg_off[gb - pa.job[j].blk0] = (long long)(inc[i] - job_off[j]);
                        start = inc[i];                   // = boff[gb - gb0]
                    }
                }
            }
        }
        // the block the next pass begins in may have begun in this one
        const int gb1 = (pass + per_pass) / BH;
        const int carry_off = boff[gb1 - gb0];
        consumer_sync<G::kConsumers>();
        if (tid == 0) {
            *carry += tot;
            boff[0] = carry_off;
        }
#pragma unroll
        for (int i = 0; i < kScanRun; ++i) c[i] = nxt[i];
        // (no barrier here: what thread 0 just wrote is read after the next pass's first barrier)
    }
    if (tid == 0) *pa.done = 0u;
}

// Per-thread counter fields -> the CTA's shared histogram: the fields are summed over the warp, the
// superset sums inverted (see count_codes_overlaid) and the per-value counts added by lane 0.
template <int N>
__device__ __forceinline__ void flush_code_counts(uint32_t (&cnt2)[HistRegs<N>::v], int left, int *s_hist) {
    constexpr int FULL = (1 << N) - 1;
    const int lane = threadIdx.x & 31;
    int f[1 << N];
#pragma unroll
    for (int m = 0; m <= FULL; ++m)
        f[m] = (int)__reduce_add_sync(kFull, (cnt2[m >> 1] >> (16 * (m & 1))) & 0xFFFFu);
    // f[FULL] holds the escapes x(0); f(full) follows from x(0) = sum_m (-1)^|m| f(m)
    int alt = 0;
#pragma unroll
    for (int m = 0; m < FULL; ++m) alt += (__builtin_popcount(m) & 1) ? -f[m] : f[m];
    f[FULL] = (N & 1) ? alt - f[FULL] : f[FULL] - alt;
    // inverse of the superset sums, one code bit at a time
#pragma unroll
    for (int i = 0; i < N; ++i)
#pragma unroll
        for (int m = 0; m <= FULL; ++m)
            if (!((m >> i) & 1)) f[m] -= f[m | (1 << i)];
#pragma unroll
    for (int v = 1; v <= FULL; ++v) {
        const int bin = left + v;
        if (lane == 0 && f[v] != 0 && bin >= 0 && bin < 256) atomicAdd(&s_hist[bin], f[v]);
    }
#pragma unroll
    for (int v = 0; v < HistRegs<N>::v; ++v) cnt2[v] = 0;
}

// FULL: the unit has G::kUnit elements (every thread has both of its chunks), so nothing is predicated.
template <int N, bool HIST, class G, bool FULL>
__device__ __forceinline__ void pack_unit(PackSmemT<G> &s, const PackStageT<G> &st, const PackUnitMeta &m,
                                          uint64_t *empty_bar, int &running, uint32_t (&cnt2)[HistRegs<N>::v],
                                          bool broken) {
    constexpr int CB = 2 * N;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // (m lives in the description ring: its destination fields are read where the unit is stored)
    if (m.first_unit_of_tile) running = 0;
    const int chunks = FULL ? G::kUnit / 16 : m.elems >> 4;

    uint4 smv[kPCPT];
    uint32_t g[kPCPT * 2], zm[kPCPT][2];
    int zc[kPCPT];
#pragma unroll
    for (int k = 0; k < kPCPT; ++k) {
        const int c = warp * (kPCPT * 32) + k * 32 + lane;
        const bool valid = FULL || c < chunks;
        uint4 w0 = make_uint4(0, 0, 0, 0), w1 = w0;
        if (valid) {
            const uint4 *p = reinterpret_cast<const uint4 *>(st.in + c * 16);
            w0 = p[0];
            w1 = p[1];
        }
        const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        uint32_t smw[4];
        uint32_t gg[2] = {0u, 0u};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            // four elements: their low bytes [e0 m6..m0] and high bytes [s e7..e1]
            const uint32_t lo4 = __byte_perm(w[2 * q], w[2 * q + 1], 0x6420);
            const uint32_t hi4 = __byte_perm(w[2 * q], w[2 * q + 1], 0x7531);
            smw[q] = (hi4 & 0x80808080u) | (lo4 & 0x7F7F7F7Fu);
            const uint32_t e4 = ((hi4 & 0x7F7F7F7Fu) << 1) | ((lo4 >> 7) & 0x01010101u);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t code = s.lut[__byte_perm(e4, 0u, 0x4440 | j)];     // byte j of e4; 0 when out of the window
                const int el = 4 * q + j;
                gg[el >> 3] = code * (1u << ((7 - (el & 7)) * N)) + gg[el >> 3];
            }
        }
        g[2 * k] = valid ? gg[0] : 0u;
        g[2 * k + 1] = valid ? gg[1] : 0u;
        zm[k][0] = valid ? zero_slots<N>(gg[0]) : 0u;
        zm[k][1] = valid ? zero_slots<N>(gg[1]) : 0u;
        zc[k] = __popc(zm[k][0]) + __popc(zm[k][1]);
        smv[k] = make_uint4(smw[0], smw[1], smw[2], smw[3]);
    }
    if (HIST) {
        count_codes_overlaid<N, kPCPT * 2>(g, cnt2);
        const int first = warp * (kPCPT * 32) + lane;
        const int mine = FULL ? 32 : (first < chunks ? 16 : 0) + (first + 32 < chunks ? 16 : 0);  // elements this thread encoded
        bump_field<N>(cnt2, 0, (uint32_t)mine);
        bump_field<N>(cnt2, (1 << N) - 1, (uint32_t)(zc[0] + zc[1]));
    }

    int incl[kPCPT];
    const int wtot = warp_scan_counts(zc, incl);
    if (lane == 0) s.warp_tot[warp] = wtot;
    bulk_wait_read();      // the previous unit's stores have finished reading the out buffers
    consumer_sync<G::kConsumers>();
    int wprefix, unit_tot;
    cross_warp_prefix<G::kWarps>(s.warp_tot, wprefix, unit_tot);
    static_assert(kPCPT == 2, "the escape loop below walks the two chunks of a thread together");
    const int c0 = warp * (kPCPT * 32) + lane;
#pragma unroll
    for (int k = 0; k < kPCPT; ++k) {
        const int c = c0 + k * 32;
        if (FULL || c < chunks) {
            *reinterpret_cast<uint4 *>(s.sm + c * 16) = smv[k];
            const uint32_t gg[2] = {g[2 * k], g[2 * k + 1]};
            store_chunk_codes<N, 16>(s.codes + c * CB, gg);
        }
    }
    if (zc[0] + zc[1] != 0) {
        // One loop over the escapes of both chunks (see unpack_unit): chunk 0 elements 0..15, then
        // chunk 1 elements 0..15, from the most significant bit of the mask.
        uint32_t todo = (compress_slots<N>(zm[0][0]) << 24) | (compress_slots<N>(zm[0][1]) << 16) |
                        (compress_slots<N>(zm[1][0]) << 8) | compress_slots<N>(zm[1][1]);
        uint8_t *out = s.esc + wprefix + incl[0] - zc[0];
        const int skip = incl[1] - zc[1] - incl[0];        // from chunk 0's escape bytes to chunk 1's
        const uint16_t *src = st.in + c0 * 16;
        int n = 0;
        while (todo) {
            const int i = __clz(todo);
            todo &= ~(0x80000000u >> i);
            // chunk 1 lies 32 chunks = 512 elements further on
            const uint32_t e = (src[((i >> 4) << 9) | (i & 15)] >> 7) & 0xFFu;
            out[n + (i >> 4) * skip] = (uint8_t)e;
            ++n;
        }
    }
    mbar_arrive(empty_bar);
    fence_async_smem();
    consumer_sync<G::kConsumers>();
    running += unit_tot;
    if (tid == 0 && !broken) {
        if (m.elems > 0) {
            bulk_store(m.sm_dst, s.sm, (uint32_t)m.elems);
            bulk_store(m.code_dst, s.codes, (uint32_t)m.elems * N / 8);
            if (unit_tot > 0) bulk_store(m.esc_dst, s.esc, (uint32_t)((unit_tot + 15) & ~15));
            bulk_commit();
        }
        *m.unit_count = unit_tot;
        if (m.last_unit_of_tile) *m.tile_count = running;
    }
}

template <int N, bool HIST, class G>
__global__ void __launch_bounds__(G::kThreads, G::kCtasPerSm) k_pack_pipe(const __grid_constant__ PackPipeArgs pa) {
    static_assert(G::kConsumers >= 256, "the 256-entry tables are filled by one consumer thread per entry");
    extern __shared__ __align__(128) uint8_t smem_raw[];
    PackSmemT<G> &s = *reinterpret_cast<PackSmemT<G> *>(smem_raw);
    const int tid = threadIdx.x;
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], G::kConsumers);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (HIST && tid < 256) s.hist[tid] = 0;
    if (tid < 2 * kStages) {
        // an empty unit: what a consumer sees if it gives up waiting before the first description is written
        PackUnitMeta &m = s.meta_ring[tid];
        m.sm_dst = m.code_dst = m.esc_dst = nullptr, m.unit_count = m.tile_count = nullptr;
        m.elems = 0, m.first_unit_of_tile = 1, m.last_unit_of_tile = 0, m.job = 0;
    }
    __syncthreads();
    // launched as a programmatic dependent of its predecessor in the stream: no global memory is touched above
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const int unit_rows = pa.unit_rows, upt = pa.units_per_tile;

    if (tid >= G::kConsumers) {
        // ---------------- producer warp ----------------
        const int lane = tid & 31;
        uint32_t it = 0;
        for (int64_t tile = blockIdx.x; tile < pa.n_tiles; tile += gridDim.x) {
            const int j = job_of_tile(pa, tile);
            const PackJob &jb = pa.job[j];
            const int64_t lt = tile - jb.tile0;
            const int64_t blk = lt / pa.BH;
            const int bh = (int)(lt - blk * pa.BH);
            const int b = bh / pa.H, h = bh - b * pa.H;
            const uint16_t *tsrc = jb.src + (int64_t)b * jb.sb + (int64_t)h * jb.sh + blk * pa.seq_tile * jb.ss;
            const bool rows_contig = (jb.ss == pa.D);
            for (int u = 0; u < upt; ++u, ++it) {
                const int stg = it % kStages;
                PackStageT<G> &st = s.stage[stg];
                mbar_wait(&s.empty[stg], ((it / kStages) & 1) ^ 1, pa.status, pa.poll_limit);
                const int row0 = u * unit_rows;
                const int rows = min(unit_rows, pa.seq_tile - row0);
                const int elems = rows * pa.D;
                if (lane == 0) {
                    PackUnitMeta &m = s.meta_ring[it % (2 * kStages)];
                    const int64_t e0 = lt * pa.tile_elems + (int64_t)row0 * pa.D;
                    m.sm_dst = jb.sign_mant + e0;
                    m.code_dst = jb.codes + e0 * N / 8;
                    m.esc_dst = pa.esc_scratch + tile * pa.tile_elems + (int64_t)row0 * pa.D;
                    m.unit_count = pa.unit_counts + tile * upt + u;
                    m.tile_count = pa.tile_counts + tile;
                    m.elems = elems;
                    m.first_unit_of_tile = (u == 0);
                    m.last_unit_of_tile = (u == upt - 1);
                    m.job = j;
                    mbar_arrive_expect_tx(&s.full[stg], (uint32_t)elems * 2u);
                }
                __syncwarp();
                const uint16_t *usrc = tsrc + (int64_t)row0 * jb.ss;
                if (rows_contig) {
                    if (lane == 0) bulk_load(st.in, usrc, (uint32_t)elems * 2u, &s.full[stg]);
                } else {
                    for (int r = lane; r < rows; r += 32)
                        bulk_load(st.in + r * pa.D, usrc + (int64_t)r * jb.ss, (uint32_t)pa.D * 2u, &s.full[stg]);
                }
            }
        }
        // do not leave while a copy into this CTA's shared memory may still be in flight (see k_unpack_pipe)
        if (launch_timed_out(pa.status))
            for (uint32_t k = it > kStages ? it - kStages : 0; k < it; ++k)
                mbar_wait(&s.full[k % kStages], (k / kStages) & 1, pa.status, pa.poll_limit);
        return;
    }

    // ---------------- consumer warps ----------------
    const int lane = tid & 31;
    uint32_t cnt2[HistRegs<N>::v];
#pragma unroll
    for (int v = 0; v < HistRegs<N>::v; ++v) cnt2[v] = 0;
    int running = 0;
    bool broken = false;                  // a wait of this warp ran out: compute on, store nothing
    int cur_job = -1, cur_left = 0;
    // (the consumers only count units: which tile a unit belongs to is in its description)
    const uint32_t my_units =
        pa.n_tiles > (int64_t)blockIdx.x
            ? (uint32_t)((pa.n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x) * (uint32_t)upt
            : 0u;
    // Units of one job run in an inner loop of their own; this outer loop only takes over when the
    // job (and with it the window and the histogram) changes.
    auto wait_loaded = [&](uint32_t u) {
        bool loaded = true;
        if (lane == 0) loaded = mbar_wait(&s.full[u % kStages], (u / kStages) & 1, pa.status, pa.poll_limit);
        loaded = __shfl_sync(kFull, loaded, 0);
        __syncwarp();      // orders the other lanes' reads of the stage after lane 0's wait
        return loaded;
    };
    uint32_t it = 0;
    while (it < my_units) {
        broken |= !wait_loaded(it);               // returns at once if the inner loop waited already
        const int job = s.meta_ring[it % (2 * kStages)].job;
        if (job != cur_job) {
            // Uniform over the CTA (every consumer reads the same sequence of units): hand the finished
            // job's histogram over and build the new job's code table.  The previous unit ended with
            // a consumer barrier, so nobody still encodes with the old table.
            if (HIST && cur_job >= 0) flush_code_counts<N>(cnt2, cur_left, s.hist);
            consumer_sync<G::kConsumers>();
            if (HIST && cur_job >= 0 && tid < 256) {
                const int hv = s.hist[tid];
                if (hv != 0 && pa.job[cur_job].hist) atomicAdd(pa.job[cur_job].hist + tid, hv);
                s.hist[tid] = 0;
            }
            cur_job = job;
            cur_left = pa.job[job].left;
            if (tid < 256) {
                const uint32_t code = (uint32_t)tid - (uint32_t)cur_left;
                s.lut[tid] = (uint8_t)(code > ((1u << N) - 1u) ? 0u : code);
            }
            consumer_sync<G::kConsumers>();
        }
        for (;;) {
            const int stg = it % kStages;
            const PackUnitMeta &meta = s.meta_ring[it % (2 * kStages)];
            if (meta.elems == G::kUnit) pack_unit<N, HIST, G, true>(s, s.stage[stg], meta, &s.empty[stg], running, cnt2, broken);
            else pack_unit<N, HIST, G, false>(s, s.stage[stg], meta, &s.empty[stg], running, cnt2, broken);
            // the per-thread counters are 16-bit fields and grow by at most 32 per unit
            if (HIST && (it & 1023u) == 1023u) flush_code_counts<N>(cnt2, cur_left, s.hist);
            if (++it >= my_units) break;
            broken |= !wait_loaded(it);
            if (s.meta_ring[it % (2 * kStages)].job != cur_job) break;
        }
    }
    if (HIST && cur_job >= 0) {
        flush_code_counts<N>(cnt2, cur_left, s.hist);
        consumer_sync<G::kConsumers>();
        if (tid < 256) {
            const int hv = s.hist[tid];
            if (hv != 0 && pa.job[cur_job].hist) atomicAdd(pa.job[cur_job].hist + tid, hv);
        }
    }
    bulk_wait_all();
    // the compaction pass may be set up from here on (it waits for this launch to complete before it reads)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __threadfence();
    consumer_sync<G::kConsumers>();
    if (tid == 0) {
        const unsigned ticket = atomicAdd(pa.done, 1u);
        s.is_last = (ticket == gridDim.x - 1);
    }
    consumer_sync<G::kConsumers>();
    if (!s.is_last) return;
    __threadfence();
    // (the staging buffers are idle by now: every unit of this CTA has been consumed and stored)
    scan_tile_counts<G>(pa, &s.carry, s.scan, s.job_off, reinterpret_cast<long long *>(&s.stage[0]));
}

// One warp copies the escape bytes of tile t (its units follow each other in the scratch) to `dst`
// of its job's stream.  The bytes move as aligned 32-bit words: the source words are funnel-shifted
// into the alignment of the destination; only the first and last word of a run use byte stores.
// With do_hist the escaped exponents are counted into `my_hist` (256 bins in shared memory).
__device__ __forceinline__ void compact_tile_units(const PackPipeArgs &pa, const PackJob &jb, int64_t t, int64_t dst,
                                                   int c, int *my_hist, bool do_hist) {
    const int lane = threadIdx.x & 31;
    const int upt = pa.units_per_tile;
    const int unit_elems = pa.unit_rows * pa.D;
    const bool fits = dst >= 0 && dst + c <= jb.capacity;
    if (!fits && lane == 0) atomicOr(pa.status, ADACODE_STATUS_ESCAPE_OVERFLOW);
    for (int u = 0; u < upt; ++u) {
        const int cu = __ldcg(pa.unit_counts + t * upt + u);
        // unit slots start on 16-byte boundaries
        const uint32_t *src4 =
            reinterpret_cast<const uint32_t *>(pa.esc_scratch + t * pa.tile_elems + (int64_t)u * unit_elems);
        uint8_t *d8 = jb.escapes + dst;
        const int r = (int)((uintptr_t)d8 & 3);
        uint32_t *dst32 = reinterpret_cast<uint32_t *>(d8 - r);
        const int n_words = (r + cu + 3) >> 2;             // destination words touched
        // four destination words (16 bytes) per lane and step: one 16-byte load of the source
        // words behind them plus the word before (for the shift)
        const uint4 *src16 = reinterpret_cast<const uint4 *>(src4);
        const int n_quads = (n_words + 3) >> 2;
#pragma unroll 2
        for (int q = lane; q < n_quads; q += 32) {
            const uint4 cur = 16 * q < cu ? __ldcg(src16 + q) : make_uint4(0u, 0u, 0u, 0u);
            const uint32_t prev = (r != 0 && q > 0) ? __ldcg(src4 + 4 * q - 1) : 0u;
            const uint32_t w[5] = {prev, cur.x, cur.y, cur.z, cur.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int j = 4 * q + k;                       // destination word
                const int s0 = 4 * j - r;                      // source index of the byte that lands in its byte 0
                const uint32_t v = r != 0 ? __funnelshift_r(w[k], w[k + 1], 8 * (4 - r)) : w[k + 1];
                if (fits && j < n_words) {
                    if (s0 >= 0 && s0 + 4 <= cu) {
                        dst32[j] = v;
                    } else {
#pragma unroll
                        for (int b = 0; b < 4; ++b)
                            if (s0 + b >= 0 && s0 + b < cu)
                                reinterpret_cast<uint8_t *>(dst32 + j)[b] = (uint8_t)(v >> (8 * b));
                    }
                }
                if (do_hist) {
                    // source word j holds source bytes 4j .. 4j+3: each source byte is counted once
                    uint32_t x = w[k + 1];
#pragma unroll
                    for (int b = 0; b < 4; ++b) {
                        if (4 * j + b < cu) atomicAdd(my_hist + (x & 0xFFu), 1);
                        x >>= 8;
                    }
                }
            }
        }
        dst += cu;
    }
}

// Gather every unit's escape bytes from its scratch slot into the compact per-segment stream.
// Tile t of global block i starts at blk_off[i] - blk_off[first block of the job] + tile_base[t] -
// count[t] in its job's stream.  blockIdx.y is the job; one warp per tile; all of a tile's metadata
// is fetched with independent loads (one memory round trip).
// With HIST the escaped exponents are counted here (whole warps of escape bytes) rather than one
// by one inside the pack kernel.  Escaped exponents cluster on a few values, so each warp keeps
// four copies of the 256 bins (picked by lane & 3): one copy would serialise most of a warp's
// shared-memory atomics.
template <bool HIST>
__global__ void __launch_bounds__(kThreads) k_compact_units(const __grid_constant__ PackPipeArgs pa) {
    __shared__ int s_hist[HIST ? kWarps : 1][HIST ? 4 : 1][HIST ? 256 : 1];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const PackJob &jb = pa.job[blockIdx.y];
    int32_t *hist = jb.hist;
    const bool do_hist = HIST && hist != nullptr;
    if (HIST) {
        for (int i = tid; i < kWarps * 4 * 256; i += kThreads) (&s_hist[0][0][0])[i] = 0;
        __syncthreads();
    }
    // launched as a programmatic dependent of the pack kernel: nothing that kernel wrote is read above
    asm volatile("griddepcontrol.wait;" ::: "memory");
    int *my_hist = &s_hist[HIST ? warp : 0][HIST ? (lane & 3) : 0][0];
    const int64_t warp_global = (int64_t)blockIdx.x * kWarps + warp;
    const int64_t n_warps = (int64_t)gridDim.x * kWarps;
    const int64_t job_tiles = (int64_t)jb.n_blocks * pa.BH;
    const int64_t job_off = __ldg(pa.blk_off + jb.blk0);
    for (int64_t lt = warp_global; lt < job_tiles; lt += n_warps) {
        const int64_t t = jb.tile0 + lt;
        // independent loads: one round trip
        const int c = __ldg(pa.tile_counts + t);
        const int tb = __ldg(jb.tile_base + lt);
        const int64_t so = __ldg(pa.blk_off + t / pa.BH) - job_off;
        if (c == 0) continue;
        compact_tile_units(pa, jb, t, so + tb - c, c, my_hist, do_hist);
    }
    if (do_hist) {
        __syncthreads();
        int total = 0;
#pragma unroll
        for (int i = 0; i < kWarps; ++i)
            total += s_hist[i][0][tid] + s_hist[i][1][tid] + s_hist[i][2][tid] + s_hist[i][3][tid];
        if (total != 0) atomicAdd(hist + tid, total);
    }
}

#endif  // ADACODE_PIPELINE_UNPACK_ONLY
