// tcgen05 decode-matmul kernel (fp16 family, every batch size).
//
// The decoded weights are the A operand of tcgen05.mma and never touch shared memory: each
// decoder thread owns one output row, decodes that row's codes in registers and writes
// them into tensor memory with tcgen05.st; the activations are the B operand, staged in
// shared memory in the canonical no-swizzle K-major layout; accumulators live in TMEM.
//
// Two operand policies share the kernel:
//   PolF8   (batch <= 8)  weights as fp6 E2M3 bytes (sign << 5 | |q|, value q/8: exact, and
//                         produced by the table XOR alone, 6 instructions per code), the
//                         fp16 activations split EXACTLY into four E5M2 planes (the top byte
//                         of the half, then of the remainder, ...), kind::f8f6f4, K = 32.
//                         The four planes are stacked along the MMA n dimension (n = 8*plane
//                         + batch column, N = 32), so one MMA per k-tile does all of them and
//                         the epilogue adds the four column groups.  The decode, the actual
//                         limiter of a 2-bit-per-weight stream, is at its minimum.
//   PolF16  (batch >= 9)  weights as fp16 integers q (byte -> half by magic number),
//                         activations as fp16, kind::f16, K = 16.
//
// Work decomposition.  A super-tile is 16 strips = 256 output rows = two M=128 MMA tiles:
// tile 0 holds strip rows 0..7 (h = 0) and tile 1 strip rows 8..15 (h = 1) of the 16 strips,
// because one 16-byte piece of the tiled code stream holds the codes of rows g and g+8 and a
// thread decodes both.  A "tile" of work is (super-tile, k-tile): 2 KiB of codes.  Tiles are
// numbered super-tile-major and split evenly and contiguously over the CTAs (stream-K); the
// part of a super-tile a CTA owns is a segment.
//
// Warp roles (22 warps):
//   0..15  decoders, four groups of four warps.  Group q takes chunks q, q+4, ... (C tiles
//          each) of a segment.  Warp wq of a group owns TMEM lanes 32wq..32wq+31 = strips
//          4wq..4wq+3; it streams its own strips through a private TMA ring, decodes, writes
//          A stage buffers in TMEM and signals its MMA issuer.  Groups 0 and 1 also run the
//          epilogue of tile 0 and tile 1.
//   16..19 MMA issuers (one thread each); issuer s serves the decoder groups q with
//          q % kNAcc == s and owns accumulator s of both MMA tiles.  Warp 16 also allocates
//          the tensor memory.
//   20..21 activation loaders.
// Every wait is bounded (mbar_wait); nothing spins on another CTA.
#pragma once
#include "dmm_common.cuh"
#include "dmm_launch.h"

namespace dmm {

// ------------------------------- tcgen05 wrappers -------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(
            taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem descriptor]
__device__ __forceinline__ void mma_ts_f16(uint32_t d, uint32_t a, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d),
        "r"(a), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void mma_ts_f8(uint32_t d, uint32_t a, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d),
        "r"(a), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
}
// Shared-memory operand descriptor, no swizzle, K-major: 8-row x 16-byte core matrices;
// lbo = byte distance between core matrices along K, sbo = between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16) |
           (static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts64(uint32_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.shared.v2.u32 [%0], {%1,%2};" ::"r"(addr), "r"(a), "r"(b) : "memory");
}

// ----------------------------------- policies -----------------------------------------
struct PolF8 {
    static constexpr int kIsF8 = 1;
    static constexpr int kFmt = kFmtFp6;
    static constexpr int kC = 4;       // tiles per chunk (= TMEM A stages per group)
    static constexpr int kNA = 4;
    static constexpr int kRing = 3;    // chunks in flight per decoder warp
    static constexpr int kACols = 8;   // TMEM columns of one A stage of one MMA tile (32 k x 1 byte)
    static constexpr int kXS = 32;     // activation stages
    static constexpr uint32_t x_stage_bytes(int) { return 1024; }  // 2 k-halves x (4 planes x 8 rows) x 16 B
    static constexpr int out_cols(int) { return 8; }                // batch columns per launch
};
struct PolF16 {
    static constexpr int kIsF8 = 0;
    static constexpr int kFmt = kFmtOffset;
    static constexpr int kC = 2;
    static constexpr int kNA = 2;
    static constexpr int kRing = 6;
    static constexpr int kACols = 16;  // 32 k x 2 bytes
    static constexpr int kXS = 12;
    static constexpr uint32_t x_stage_bytes(int nmma) { return static_cast<uint32_t>(nmma) * 64u; }  // 4 k-chunks x rows x 16 B
    static constexpr int out_cols(int nmma) { return nmma; }
};

constexpr int kUDecWarps = 16, kUMmaWarp = 16, kUMmaWarps = 4, kULoadWarps = 2;
constexpr int kUThreads = (kUDecWarps + kUMmaWarps + kULoadWarps) * 32;
constexpr uint32_t kUBarBytes = 2048;
constexpr uint32_t kUTmemCols = 512;

template <class Pol, int NMMA>
struct UmmaPlan {
    static constexpr int kNAcc = NMMA <= 32 ? 4 : 2;             // accumulators per MMA tile
    static constexpr uint32_t kDCols = 2 * kNAcc * NMMA;         // TMEM: accumulators first
    static constexpr uint32_t kACols = 4 * Pol::kNA * 2 * Pol::kACols;
    static_assert(kDCols + kACols <= kUTmemCols, "TMEM plan exceeds 512 columns");
    static constexpr uint32_t kXStage = Pol::x_stage_bytes(NMMA);
    static constexpr uint32_t kXBytes = Pol::kXS * kXStage;
    static constexpr int kNB = Pol::out_cols(NMMA);               // output columns per launch
    static constexpr uint32_t kPreBytes = kUBarBytes + kXBytes;
    static constexpr uint32_t kSlotBytes = 4 * Pol::kC * 128;    // 4 strips x C k-tiles
    static constexpr uint32_t kRingBytes = kUDecWarps * Pol::kRing * kSlotBytes;
    static constexpr uint32_t kDynBytes = 0x10000u - 0x400u + kLutBytes + kRingBytes;
    static constexpr int kPartial = 2 * kNB * 128;               // output values per segment
    static_assert(kPreBytes <= 0x10000u - 0x400u, "activation stages do not fit below the table");
    static_assert(kDynBytes <= 232448u, "shared memory plan exceeds the per-CTA limit");
    // barrier indices
    static constexpr int kBarCode = 0;                                   // [16][kRing]
    static constexpr int kBarAFull = kBarCode + kUDecWarps * Pol::kRing;  // [4][kNA]
    static constexpr int kBarAFree = kBarAFull + 4 * Pol::kNA;
    static constexpr int kBarXFull = kBarAFree + 4 * Pol::kNA;           // [kXS]
    static constexpr int kBarXFree = kBarXFull + Pol::kXS;
    static constexpr int kBarDReady = kBarXFree + Pol::kXS;
    static constexpr int kBarDFree = kBarDReady + 1;
    static constexpr int kBarCount = kBarDFree + 1;
    static_assert(kBarCount * 8 + 64 <= kUBarBytes, "barrier block too small");
};

struct UmmaParams {
    const void *x;       // [M, K] fp16
    const void *codes;   // tiled codes
    const void *cb;      // fp16 [256, 8]
    float *out;          // [M, N]
    float *partials;     // workspace [grid][2][kPartial]
    unsigned *tickets;   // workspace, one per super-tile, zero between launches
    long long M, N, K;
    float scale;         // includes the unit of the accumulators (1/4 for q, 2 for q/8)
    int accumulate;
    int sign_convention;
    unsigned dyn_smem_bytes;
};

template <class Pol, int NMMA>
__global__ void __launch_bounds__(kUThreads, 1) umma_kernel(const UmmaParams p) {
    using Plan = UmmaPlan<Pol, NMMA>;
    constexpr int C = Pol::kC, NA = Pol::kNA, RING = Pol::kRing, XS = Pol::kXS, NACC = Plan::kNAcc, NB = Plan::kNB;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t lut_addr = (base + Plan::kPreBytes + 0xFFFFu) & ~0xFFFFu;
    const uint32_t ring_addr = lut_addr + kLutBytes;
    const uint32_t x_addr = base + kUBarBytes;
    volatile int *flags = reinterpret_cast<volatile int *>(smem_raw + Plan::kBarCount * 8);  // [0]=failed [1]=last
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_raw + Plan::kBarCount * 8 + 16);
    auto bar = [&](int i) -> uint32_t { return base + 8u * static_cast<uint32_t>(i); };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (ring_addr + Plan::kRingBytes > base + p.dyn_smem_bytes) {  // uniform over the grid
        if (tid == 0) raise_status(DMM_STATUS_BAD_SMEM);
        return;
    }

    const int KT = static_cast<int>(p.K / 32);
    const int NS = static_cast<int>(p.N / 16);
    const int SST = (NS + 15) / 16;  // super-tiles
    const long long T = static_cast<long long>(SST) * KT;
    const long long G = gridDim.x, cta = blockIdx.x;
    const long long i0 = part_begin(T, G, cta), i1 = part_begin(T, G, cta + 1);
    const int ss_first = static_cast<int>(i0 / KT), ss_last = static_cast<int>((i1 - 1) / KT);
    auto seg_begin = [&](int ss) -> long long {
        const long long a = static_cast<long long>(ss) * KT;
        return i0 > a ? i0 : a;
    };
    auto seg_len = [&](int ss) -> int {
        const long long a = static_cast<long long>(ss) * KT;
        const long long lo = i0 > a ? i0 : a, hi = i1 < a + KT ? i1 : a + KT;
        return static_cast<int>(hi - lo);
    };

    // ---- set-up: barriers, TMEM, zeroed activation stages ----
    if (tid == 0) {
        for (int i = 0; i < kUDecWarps * RING; ++i) mbar_init(bar(Plan::kBarCode + i), 1);
        for (int i = 0; i < 4 * NA; ++i) {
            mbar_init(bar(Plan::kBarAFull + i), 4);
            mbar_init(bar(Plan::kBarAFree + i), 1);
        }
        for (int i = 0; i < XS; ++i) {
            mbar_init(bar(Plan::kBarXFull + i), 1);
            mbar_init(bar(Plan::kBarXFree + i), 1);
        }
        mbar_init(bar(Plan::kBarDReady), NACC);
        mbar_init(bar(Plan::kBarDFree), 8);
        flags[0] = 0;
        flags[1] = 0;
        fence_mbar_init();
    }
    if (warp == kUMmaWarp) tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kUTmemCols);
    for (uint32_t o = tid * 16u; o < Plan::kXBytes; o += kUThreads * 16u) sts128(x_addr + o, make_uint4(0, 0, 0, 0));
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    grid_dep_launch();

    if (warp < kUDecWarps) {
        // =============================== decoders ===============================
        const int q = warp >> 2, wq = warp & 3;
        const uint32_t wring = ring_addr + static_cast<uint32_t>(warp) * (RING * Plan::kSlotBytes);
        const uint64_t policy = policy_evict_first();
        const uint8_t *codes = reinterpret_cast<const uint8_t *>(p.codes);

        struct Cur {
            int ss, c;
            bool ok;
        };
        auto settle = [&](Cur &cu) {  // first chunk of group q at or after (ss, c)
            while (cu.ok && cu.c * C >= seg_len(cu.ss)) {
                if (cu.ss == ss_last) {
                    cu.ok = false;
                } else {
                    ++cu.ss;
                    cu.c = q;
                }
            }
        };
        auto issue = [&](const Cur &cu, int idx) {
            const int len = seg_len(cu.ss);
            const int n = len - cu.c * C < C ? len - cu.c * C : C;
            const int kt = static_cast<int>(seg_begin(cu.ss) - static_cast<long long>(cu.ss) * KT) + cu.c * C;
            const int strip = cu.ss * 16 + wq * 4 + lane;  // lanes 0..3
            const int nvalid = NS - (cu.ss * 16 + wq * 4);  // strips of this warp that exist
            const int ns = nvalid < 0 ? 0 : (nvalid > 4 ? 4 : nvalid);
            const uint32_t b = bar(Plan::kBarCode + warp * RING + idx % RING);
            if (lane == 0) mbar_arrive_expect_tx(b, static_cast<uint32_t>(n * 128 * ns));
            __syncwarp();
            if (lane < ns)
                bulk_g2s(wring + (idx % RING) * Plan::kSlotBytes + lane * (C * 128),
                         codes + (static_cast<long long>(strip) * KT + kt) * 128, static_cast<uint32_t>(n * 128), b,
                         policy);
        };

        Cur icur{ss_first, q, true}, ccur;
        settle(icur);
        ccur = icur;
        int iidx = 0, cidx = 0;
        while (iidx < RING && icur.ok) {  // weights do not depend on the previous kernel
            issue(icur, iidx);
            icur.c += 4;
            settle(icur);
            ++iidx;
        }

        const bool bad = lut_fill(lut_addr, p.cb, 1, p.sign_convention, Pol::kFmt, tid, kUDecWarps * 32);
        if (bad) raise_status(DMM_STATUS_BAD_CODEBOOK);
        named_barrier(1, kUDecWarps * 32);
        const LutLane ll = lut_lane(lut_addr, lane);
        grid_dep_wait();

        const uint32_t tlane = tmem + (static_cast<uint32_t>(wq * 32) << 16);
        const uint32_t a_base = Plan::kDCols + static_cast<uint32_t>(q * NA) * 2 * Pol::kACols;
        uint32_t sA = 0;
        int segidx = 0;
        for (int ss = ss_first; ss <= ss_last; ++ss, ++segidx) {
            while (ccur.ok && ccur.ss == ss) {
                const int len = seg_len(ss);
                const int n = len - ccur.c * C < C ? len - ccur.c * C : C;
                const int slot = cidx % RING;
                mbar_wait(bar(Plan::kBarCode + warp * RING + slot), static_cast<uint32_t>((cidx / RING) & 1), flags);
                const uint32_t src = wring + slot * Plan::kSlotBytes + (lane >> 3) * (C * 128) + (lane & 7) * 16;
                for (int i = 0; i < n; ++i) {
                    const int buf = static_cast<int>(sA % NA);
                    if (sA >= NA) mbar_wait(bar(Plan::kBarAFree + q * NA + buf), ((sA / NA) - 1) & 1, flags);
                    tc_fence_after();
                    const uint4 cw = lds128(src + i * 128);
                    const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
                    const uint32_t acol = tlane + a_base + static_cast<uint32_t>(buf) * 2 * Pol::kACols;
                    if constexpr (Pol::kIsF8) {
                        uint32_t r0[8], r1[8];
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            const uint2 d0 = decode8<0>(w[t], ll), d1 = decode8<1>(w[t], ll);
                            r0[2 * t] = d0.x; r0[2 * t + 1] = d0.y;
                            r1[2 * t] = d1.x; r1[2 * t + 1] = d1.y;
                        }
                        tmem_st8(acol, r0);
                        tmem_st8(acol + Pol::kACols, r1);
                    } else {
                        uint32_t r0[16], r1[16];
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            uint32_t h0[4], h1[4];
                            bytes_to_half2(decode8<0>(w[t], ll), h0);
                            bytes_to_half2(decode8<1>(w[t], ll), h1);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                r0[4 * t + e] = h0[e];
                                r1[4 * t + e] = h1[e];
                            }
                        }
                        tmem_st16(acol, r0);
                        tmem_st16(acol + Pol::kACols, r1);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(Plan::kBarAFull + q * NA + buf));
                    ++sA;
                }
                __syncwarp();  // every lane has read the slot: refill it
                if (icur.ok) {
                    issue(icur, iidx);
                    icur.c += 4;
                    settle(icur);
                    ++iidx;
                }
                ccur.c += 4;
                settle(ccur);
                ++cidx;
            }

            if (q < 2) {
                // ---------------- epilogue of MMA tile q of this segment ----------------
                const int len = seg_len(ss);
                const int nchunks = (len + C - 1) / C;
                const int nacc = nchunks < NACC ? nchunks : NACC;
                mbar_wait(bar(Plan::kBarDReady), static_cast<uint32_t>(segidx & 1), flags);
                tc_fence_after();
                float v[NB];
#pragma unroll
                for (int b = 0; b < NB; ++b) v[b] = 0.f;
#pragma unroll
                for (int a = 0; a < NACC; ++a) {
                    if (a < nacc) {
#pragma unroll
                        for (int b0 = 0; b0 < NMMA; b0 += 16) {
                            uint32_t r[16];
                            tmem_ld16(tlane + static_cast<uint32_t>((q * NACC + a) * NMMA + b0), r);
                            tmem_wait_ld();
                            // PolF8: column 8*plane + b; PolF16: column b
#pragma unroll
                            for (int e = 0; e < 16; ++e) v[(b0 + e) % NB] += __uint_as_float(r[e]);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(Plan::kBarDFree));

                const long long ss_a = static_cast<long long>(ss) * KT;
                const bool full = len == KT;
                const int my_slot = seg_begin(ss) > ss_a ? 0 : 1;
                const int trow = wq * 32 + lane;  // TMEM lane = row of the MMA tile
                const long long n = (static_cast<long long>(ss) * 16 + wq * 4 + (lane >> 3)) * 16 + 8 * q + (lane & 7);
                const int ptid = q * 128 + trow;
                if (full) {
                    if (n < p.N) {
#pragma unroll
                        for (int b = 0; b < NB; ++b)
                            if (b < p.M) {
                                float *o = p.out + b * p.N + n;
                                const float r = p.scale * v[b];
                                *o = p.accumulate ? *o + r : r;
                            }
                    }
                } else {
                    float *mine = p.partials + (cta * 2 + my_slot) * Plan::kPartial + q * NB * 128 + trow;
#pragma unroll
                    for (int b = 0; b < NB; ++b)
                        if (b < p.M) mine[b * 128] = v[b];
                    __threadfence();
                    named_barrier(2, 256);
                    const long long c_lo = part_owner(T, G, ss_a), c_hi = part_owner(T, G, ss_a + KT - 1);
                    if (ptid == 0) {
                        const unsigned expected = static_cast<unsigned>(c_hi - c_lo + 1);
                        const unsigned old = atomicAdd(p.tickets + ss, 1u);
                        const int last = old == expected - 1;
                        if (last) p.tickets[ss] = 0;
                        flags[1] = last;
                    }
                    named_barrier(2, 256);
                    if (flags[1] != 0) {
                        __threadfence();
                        if (n < p.N) {
#pragma unroll
                            for (int b = 0; b < NB; ++b)
                                if (b < p.M) {
                                    float tot = 0.f;
                                    for (long long c = c_lo; c <= c_hi; ++c) {
                                        const int slot_c = part_begin(T, G, c) > ss_a ? 0 : 1;
                                        tot += __ldcg(p.partials + (c * 2 + slot_c) * Plan::kPartial + (q * NB + b) * 128 +
                                                      trow);
                                    }
                                    float *o = p.out + b * p.N + n;
                                    const float r = p.scale * tot;
                                    *o = p.accumulate ? *o + r : r;
                                }
                        }
                    }
                    named_barrier(2, 256);  // flags[1] is reused by the next segment
                }
            }
        }
    } else if (warp < kUMmaWarp + kUMmaWarps) {
        // =============================== MMA issuers ===============================
        const int me = warp - kUMmaWarp;  // accumulator index this issuer owns
        if (lane == 0 && me < NACC) {
            uint32_t cnt[4] = {0, 0, 0, 0};  // A stages consumed per decoder group (only own groups advance)
            int segidx = 0;
            const uint32_t idesc = Pol::kIsF8
                                       ? ((1u << 4) | (3u << 7) | (1u << 10) | ((NMMA >> 3) << 17) | ((128u >> 4) << 24))
                                       : ((1u << 4) | ((NMMA >> 3) << 17) | ((128u >> 4) << 24));
            // descriptor of activation stage 0; later stages and k-halves only move the address field
            const uint64_t xdesc0 = Pol::kIsF8 ? smem_desc(x_addr, 512, 128) : smem_desc(x_addr, NMMA * 16, 128);
            uint32_t xi = 0;  // CTA-wide tile counter (every issuer counts all tiles)
            for (int ss = ss_first; ss <= ss_last; ++ss, ++segidx) {
                const int len = seg_len(ss);
                if (segidx > 0) {
                    mbar_wait(bar(Plan::kBarDFree), static_cast<uint32_t>((segidx - 1) & 1), flags);
                    tc_fence_after();
                }
                uint32_t on = 0;  // accumulator already holds data of this segment
                for (int j = 0; j < len; ++j, ++xi) {
                    const int q = (j / C) & 3;
                    if (q % NACC != me) continue;
                    const uint32_t c = q < 2 ? cnt[q] : cnt[q];
                    const int buf = static_cast<int>(c % NA);
                    const uint32_t xs = xi % XS;
                    mbar_wait(bar(Plan::kBarAFull + q * NA + buf), (c / NA) & 1, flags);
                    mbar_wait(bar(Plan::kBarXFull + xs), (xi / XS) & 1, flags);
                    tc_fence_after();
                    const uint64_t xd = xdesc0 + ((xs * Plan::kXStage) >> 4);
                    const uint32_t a_col = tmem + Plan::kDCols + static_cast<uint32_t>(q * NA + buf) * 2 * Pol::kACols;
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        const uint32_t d_col = tmem + static_cast<uint32_t>((t * NACC + me) * NMMA);
                        if constexpr (Pol::kIsF8) {
                            mma_ts_f8(d_col, a_col + t * Pol::kACols, xd, idesc, on);
                        } else {
                            mma_ts_f16(d_col, a_col + t * Pol::kACols, xd, idesc, on);
                            mma_ts_f16(d_col, a_col + t * Pol::kACols + 8, xd + ((2 * NMMA * 16) >> 4), idesc, 1u);
                        }
                    }
                    on = 1;
                    tc_commit(bar(Plan::kBarAFree + q * NA + buf));
                    tc_commit(bar(Plan::kBarXFree + xs));
                    ++cnt[q];
                }
                tc_commit(bar(Plan::kBarDReady));
            }
        }
    } else {
        // =========================== activation loaders ===========================
        grid_dep_wait();
        const int wl = warp - kUMmaWarp - kUMmaWarps;
        const __half *x = reinterpret_cast<const __half *>(p.x);
        const int M = static_cast<int>(p.M);
        // CTA-wide tile stream in processing order: segment by segment, k-tile by k-tile
        int cs = ss_first, cj = 0;  // cursor: segment, tile inside it
        auto kt_of = [&](int ss, int j) -> int {
            return static_cast<int>(seg_begin(ss) - static_cast<long long>(ss) * KT) + j;
        };
        auto skip = [&](int nskip) -> bool {  // advance the cursor; false when the stream ends
            cj += nskip;
            while (cj >= seg_len(cs)) {
                if (cs == ss_last) return false;
                cj -= seg_len(cs);
                ++cs;
            }
            return true;
        };
        if constexpr (Pol::kIsF8) {
            // lanes cover (tile of the batch, piece): piece = (row, 8-k chunk)
            const int pp = M <= 1 ? 4 : M <= 2 ? 8 : M <= 4 ? 16 : 32;  // lanes per tile
            const int tb = 32 / pp;                                     // tiles per pass
            const int u_n = tb >= 4 ? 1 : 4 / tb;                       // passes per batch (loads in flight)
            const int bt = tb * u_n;                                    // tiles per batch
            const int piece = lane % pp, tsub = lane / pp;
            const int row = piece >> 2, kc = piece & 3;
            const bool active = piece < M * 4;
            bool more = skip(wl * bt);
            uint32_t xi = static_cast<uint32_t>(wl * bt);
            while (more) {
                uint4 v[4];
                bool have[4];
                uint32_t stage[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    have[u] = false;
                    if (u < u_n) {
                        // tile index inside the batch: u * tb + tsub; locate it without moving the cursor
                        int s2 = cs, j2 = cj + u * tb + tsub;
                        bool ok = true;
                        while (j2 >= seg_len(s2)) {
                            if (s2 == ss_last) { ok = false; break; }
                            j2 -= seg_len(s2);
                            ++s2;
                        }
                        const uint32_t my_xi = xi + static_cast<uint32_t>(u * tb + tsub);
                        stage[u] = my_xi % XS;
                        if (ok) {
                            if (my_xi >= XS) mbar_wait(bar(Plan::kBarXFree + stage[u]), ((my_xi / XS) - 1) & 1, flags);
                            have[u] = true;
                            if (active)
                                v[u] = __ldg(reinterpret_cast<const uint4 *>(x + static_cast<long long>(row) * p.K +
                                                                             32 * kt_of(s2, j2) + 8 * kc));
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    if (u < u_n && have[u]) {
                        if (active) {
                            uint32_t h[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
                            // stage layout [k-half][8*plane + row][16 B]
                            const uint32_t dst = x_addr + stage[u] * Plan::kXStage + (kc >> 1) * 512 + row * 16 + (kc & 1) * 8;
#pragma unroll
                            for (int pl = 0; pl < 4; ++pl) {
                                // plane pl = top byte of each half (an E5M2 number), then subtract it
                                sts64(dst + pl * 128, prmt(h[0], h[1], 0x7531u), prmt(h[2], h[3], 0x7531u));
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const uint32_t top = h[e] & 0xFF00FF00u;
                                    __half2 r = __hsub2(*reinterpret_cast<__half2 *>(&h[e]),
                                                        *reinterpret_cast<const __half2 *>(&top));
                                    h[e] = *reinterpret_cast<uint32_t *>(&r);
                                }
                            }
                        }
                        fence_async_smem();
                    }
                }
                __syncwarp();
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (u < u_n && have[u] && piece == 0) mbar_arrive(bar(Plan::kBarXFull + stage[u]));
                xi += static_cast<uint32_t>(kULoadWarps * bt);
                more = skip(kULoadWarps * bt);
            }
        } else {
            // warp wl stages tiles wl, wl+3, ...; three tiles in flight per warp
            bool more = skip(wl);
            uint32_t xi = static_cast<uint32_t>(wl);
            uint32_t pend[3] = {0, 0, 0};
            int npend = 0;
            auto retire = [&]() {  // oldest pending tile has landed
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(Plan::kBarXFull + pend[0] % XS));
                pend[0] = pend[1];
                pend[1] = pend[2];
                --npend;
            };
            while (more) {
                const uint32_t st = xi % XS;
                if (xi >= XS) mbar_wait(bar(Plan::kBarXFree + st), ((xi / XS) - 1) & 1, flags);
                const int kt = kt_of(cs, cj);
                const uint32_t dst = x_addr + st * Plan::kXStage;
                for (int pc = lane; pc < M * 4; pc += 32) {
                    const int row = pc >> 2, kc = pc & 3;
                    cp_async16(dst + kc * (NMMA * 16) + row * 16, x + static_cast<long long>(row) * p.K + 32 * kt + 8 * kc);
                }
                cp_async_commit();
                pend[npend++] = xi;
                if (npend == 3) {
                    cp_async_wait<2>();
                    retire();
                }
                xi += kULoadWarps;
                more = skip(kULoadWarps);
            }
            while (npend > 0) {
                if (npend == 3) cp_async_wait<2>(); else if (npend == 2) cp_async_wait<1>(); else cp_async_wait<0>();
                retire();
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kUMmaWarp) tmem_dealloc(tmem, kUTmemCols);
}

template <class Pol, int NMMA>
inline int launch_umma_one(const UmmaParams &p_in, int num_sms, bool pdl, cudaStream_t stream) {
    using Plan = UmmaPlan<Pol, NMMA>;
    UmmaParams p = p_in;
    p.dyn_smem_bytes = Plan::kDynBytes;
    auto kernel = umma_kernel<Pol, NMMA>;
    cudaError_t err =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Plan::kDynBytes));
    if (err != cudaSuccess) return err;
    const long long KT = p.K / 32, NS = p.N / 16, SST = (NS + 15) / 16;
    const long long T = SST * KT;
    const unsigned grid = static_cast<unsigned>(T < num_sms ? T : num_sms);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kUThreads);
    cfg.dynamicSmemBytes = Plan::kDynBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

// f8 != 0: PolF8 (needs M <= 8); else PolF16 with M <= 64.
inline int launch_umma(bool f8, const UmmaParams &p, int num_sms, bool pdl, cudaStream_t stream) {
    if (f8) return launch_umma_one<PolF8, 32>(p, num_sms, pdl, stream);
    if (p.M <= 16) return launch_umma_one<PolF16, 16>(p, num_sms, pdl, stream);
    if (p.M <= 32) return launch_umma_one<PolF16, 32>(p, num_sms, pdl, stream);
    return launch_umma_one<PolF16, 64>(p, num_sms, pdl, stream);
}

// Workspace floats per CTA slot for a batch of M columns on this path.
inline int umma_partial_values(long long M, bool f8) {
    const int nb = f8 ? 8 : (M <= 16 ? 16 : (M <= 32 ? 32 : 64));
    return 2 * nb * 128;
}

}  // namespace dmm
