// Streaming decode-matmul kernel (small-batch path, both families).
//
// One persistent CTA of NW warps per SM.  The tiled code matrix is a linear stream of
// (N/16 strips) x (K/32 k-tiles) x 128 bytes.  The unit of work is a "tile": S strips
// (a super-strip of 16*S output rows) x one k-tile (32 reduction indices), S*128 bytes of
// codes.  Tiles are numbered super-strip-major and split evenly and contiguously over the
// CTAs (stream-K), so every SM streams the same number of bytes whatever N and K are.  The
// part of a super-strip that a CTA owns (a "segment") is split evenly and contiguously over
// its warps, so all warps work on the same segment at the same time.
//
//   per warp : a private ring of D stages in shared memory.  Lanes 0..S-1 issue 1-D bulk
//              copies (TMA), one per strip, of up to C consecutive k-tiles; completion is
//              counted on the stage's mbarrier.  The warp that reads a stage is the warp
//              that refills it, so no "empty" barriers and no producer warp are needed.
//              Per k-tile and strip each lane reads one word (2 codes: rows g and g+8 of
//              the strip), decodes it with two table look-ups + XOR (dmm_common.cuh) and
//              feeds legacy warp-level MMAs whose B operand is the activation fragment
//              (batch along the MMA n dimension, 8 columns per group).
//   per CTA  : for each super-strip the CTA touches, a cross-warp reduction through shared
//              memory, then either a direct store (the CTA covered the whole K range) or a
//              partial written to the workspace; the last CTA to arrive (ticket counter)
//              sums the partials in a fixed order and stores.  No CTA waits for another.
//
// Fragment bookkeeping.  Lane l = 4g + t.  The word of a lane holds the codes of strip rows
// g (low half) and g+8 (high half) for reduction indices k = 32*kt + 8*t + i, i = 0..7.
// The MMA sums over "slots"; both operands use the same slot -> k map, so any map works:
//   fp16  m16n8k16: MMA 1 gets weights i = 0..3 (slots 2t,2t+1 | 2t+8,2t+9), MMA 2 i = 4..7.
//   int8  m16n8k32: slots 4t..4t+3 = i 0..3, slots 4t+16..4t+19 = i 4..7.
#pragma once
#include "dmm_common.cuh"
#include "dmm_launch.h"

namespace dmm {

struct FamF16 {
    using x_t = __half;
    using acc_t = float;
    static constexpr int kIsF16 = 1;
    static constexpr int kFmt = kFmtOffset;
    static constexpr int kXRegs = 4;  // 8 halfs per k-tile per lane
};

constexpr int kStreamWarps = 16;   // NW
constexpr int kChunkTiles = 4;     // C: k-tiles per bulk copy
constexpr int kStages = 3;         // D: stages per warp
constexpr uint32_t kBarBytes = 1024;

// Shared-memory map (absolute shared-window addresses; dynamic shared memory starts at
// `base`, 0x400 on sm_100):
//   base            barriers (NW*D) and flags                       kBarBytes
//   base+kBarBytes  cross-warp reduction buffer                     NW*S*MB*128*4
//   0x10000-aligned decode table                                    64 KiB
//   table+64 KiB    code ring: NW warps x D stages x S*C*128 bytes
template <int S, int MB>
struct SmemPlan {
    static constexpr uint32_t kStageBytes = S * kChunkTiles * 128;
    static constexpr uint32_t kRingBytes = kStreamWarps * kStages * kStageBytes;
    static constexpr uint32_t kRedBytes = kStreamWarps * S * MB * 128 * 4;
    static constexpr uint32_t kPreBytes = kBarBytes + kRedBytes;
    // enough when base <= 0x400 + slack: table at 0x10000
    static constexpr uint32_t kDynBytes = 0x10000u - 0x400u + kLutBytes + kRingBytes;
    static_assert(kPreBytes <= 0x10000u - 0x400u, "reduction buffer does not fit below the table");
    static_assert(kDynBytes <= 232448u, "shared memory plan exceeds the per-CTA limit");
};

// Writes accumulator value `o` of super-strip `ss` to the output matrix.
// o = ((s*MB + mb)*32 + lane)*4 + c follows the MMA accumulator fragment:
// row = lane/4 + 8*(c/2) of strip s, batch column = 8*mb + 2*(lane%4) + c%2.
template <class Fam, int S, int MB>
__device__ __forceinline__ void store_out(const StreamParams &p, long long ss, int o, typename Fam::acc_t v) {
    const int s = o / (MB * 128), mb = (o / 128) % MB, l = (o % 128) / 4, c = o % 4;
    const long long n = (ss * S + s) * 16 + (l >> 2) + 8 * (c >> 1);
    const long long col = mb * 8 + 2 * (l & 3) + (c & 1);
    if (col >= p.M || n >= p.N) return;
    float *out = reinterpret_cast<float *>(p.out) + col * p.N + n;
    const float r = p.scale * v;
    *out = p.accumulate ? *out + r : r;
}

// Position of a warp in its tile sequence: the segment (super-strip) it is in and its
// sub-range [pos, end) of global tile indices inside that segment.
struct Cursor {
    int ss;
    long long pos, end;
};

template <class Fam, int S, int MB>
__global__ void __launch_bounds__(kStreamWarps * 32, 1) stream_kernel(const StreamParams p) {
    using acc_t = typename Fam::acc_t;
    using Plan = SmemPlan<S, MB>;
    constexpr int NW = kStreamWarps, C = kChunkTiles, D = kStages;
    constexpr int XR = Fam::kXRegs;
    constexpr int PSZ = S * MB * 128;  // accumulator values per super-strip
    constexpr int kThreads = NW * 32;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t lut_addr = (base + Plan::kPreBytes + 0xFFFFu) & ~0xFFFFu;
    const uint32_t ring_addr = lut_addr + kLutBytes;
    volatile int *flags = reinterpret_cast<volatile int *>(smem_raw + NW * D * 8);  // [0]=failed [1]=last
    acc_t *red = reinterpret_cast<acc_t *>(smem_raw + kBarBytes);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (ring_addr + Plan::kRingBytes > base + p.dyn_smem_bytes) {  // uniform over the grid
        if (tid == 0) raise_status(DMM_STATUS_BAD_SMEM);
        return;
    }

    const int KT = static_cast<int>(p.K / 32);           // k-tiles per strip
    const int NS = static_cast<int>(p.N / 16);           // strips
    const int SS = (NS + S - 1) / S;                     // super-strips
    const long long T = static_cast<long long>(SS) * KT;  // tiles
    const long long G = gridDim.x;
    const long long cta = blockIdx.x;
    const long long i0 = part_begin(T, G, cta), i1 = part_begin(T, G, cta + 1);   // CTA range
    const int ss_first = static_cast<int>(i0 / KT), ss_last = static_cast<int>((i1 - 1) / KT);

    const uint32_t wbar = base + static_cast<uint32_t>(warp) * (D * 8);
    const uint32_t wring = ring_addr + static_cast<uint32_t>(warp) * (D * Plan::kStageBytes);
    if (lane == 0) {
        for (int d = 0; d < D; ++d) mbar_init(wbar + 8u * d, 1);
        if (tid == 0) {
            flags[0] = 0;
            flags[1] = 0;
        }
        fence_mbar_init();
    }
    __syncwarp();
    grid_dep_launch();

    // ---- per-warp code pipeline ----
    const uint64_t policy = policy_evict_first();
    const uint8_t *codes = reinterpret_cast<const uint8_t *>(p.codes);
    // sub-range of this warp in segment ss
    auto enter = [&](Cursor &c, int ss) {
        const long long ss_a = static_cast<long long>(ss) * KT;
        const long long seg_a = i0 > ss_a ? i0 : ss_a;
        const long long seg_b = i1 < ss_a + KT ? i1 : ss_a + KT;
        const long long len = seg_b - seg_a;
        c.ss = ss;
        c.pos = seg_a + len * warp / NW;
        c.end = seg_a + len * (warp + 1) / NW;
    };
    // skips empty sub-ranges; afterwards pos < end unless the warp's sequence is exhausted
    auto normalize = [&](Cursor &c) {
        while (c.pos == c.end && c.ss < ss_last) enter(c, c.ss + 1);
    };
    auto chunk_tiles = [&](const Cursor &c) -> int {
        const long long left = c.end - c.pos;
        return left < C ? static_cast<int>(left) : C;
    };
    auto issue = [&](const Cursor &c, int idx) {
        const int n = chunk_tiles(c);
        const int nstrips = NS - c.ss * S < S ? NS - c.ss * S : S;
        const int kt = static_cast<int>(c.pos - static_cast<long long>(c.ss) * KT);
        const uint32_t bar = wbar + 8u * (idx % D);
        if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(n * 128 * nstrips));
        __syncwarp();
        if (lane < nstrips) {
            const uint8_t *src = codes + (static_cast<long long>(c.ss * S + lane) * KT + kt) * 128;
            bulk_g2s(wring + (idx % D) * Plan::kStageBytes + lane * (C * 128), src, static_cast<uint32_t>(n * 128), bar,
                     policy);
        }
    };

    Cursor icur, ccur;
    enter(icur, ss_first);
    normalize(icur);
    ccur = icur;
    int iidx = 0, cidx = 0;
    while (iidx < D && icur.pos < icur.end) {  // weights do not depend on the previous kernel
        issue(icur, iidx);
        icur.pos += chunk_tiles(icur);
        normalize(icur);
        ++iidx;
    }

    const bool bad = lut_fill(lut_addr, p.cb, p.cb_is_f16, p.sign_convention, Fam::kFmt, tid, kThreads);
    if (bad) raise_status(DMM_STATUS_BAD_CODEBOOK);
    __syncthreads();
    const LutLane ll = lut_lane(lut_addr, lane);

    grid_dep_wait();  // activations, out (accumulate), workspace: only after the previous kernel

    const int g = lane >> 2, t = lane & 3;
    const typename Fam::x_t *x = reinterpret_cast<const typename Fam::x_t *>(p.x);

    // activation fragments of one chunk: xf[mb][jt][r], 8 consecutive k per (lane, k-tile)
    auto load_x = [&](uint32_t (&xf)[MB][C][XR], int kt0, int n) {
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
            const long long col = mb * 8 + g;
#pragma unroll
            for (int jt = 0; jt < C; ++jt) {
#pragma unroll
                for (int r = 0; r < XR; ++r) xf[mb][jt][r] = 0;
                if (col < p.M && jt < n) {
                    const typename Fam::x_t *src = x + col * p.K + 32 * (kt0 + jt) + 8 * t;
                    if constexpr (XR == 4) {
                        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(src));
                        xf[mb][jt][0] = v.x; xf[mb][jt][1] = v.y; xf[mb][jt][2] = v.z; xf[mb][jt][3] = v.w;
                    } else {
                        const uint2 v = __ldg(reinterpret_cast<const uint2 *>(src));
                        xf[mb][jt][0] = v.x; xf[mb][jt][1] = v.y;
                    }
                }
            }
        }
    };

    for (int ss = ss_first; ss <= ss_last; ++ss) {
        const long long ss_a = static_cast<long long>(ss) * KT, ss_b = ss_a + KT;
        const long long seg_a = i0 > ss_a ? i0 : ss_a;
        const long long seg_b = i1 < ss_b ? i1 : ss_b;
        const int nstrips = NS - ss * S < S ? NS - ss * S : S;

        acc_t acc[S][MB][4];
#pragma unroll
        for (int s = 0; s < S; ++s)
#pragma unroll
            for (int mb = 0; mb < MB; ++mb)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[s][mb][c] = 0;

        while (ccur.ss == ss && ccur.pos < ccur.end) {
            const int n = chunk_tiles(ccur);
            uint32_t xf[MB][C][XR];
            load_x(xf, static_cast<int>(ccur.pos - ss_a), n);

            const int slot = cidx % D;
            mbar_wait(wbar + 8u * slot, static_cast<uint32_t>((cidx / D) & 1), flags);
            const uint32_t stage = wring + slot * Plan::kStageBytes + lane * 4u;

#pragma unroll
            for (int s = 0; s < S; ++s) {
                if (s < nstrips) {
#pragma unroll
                    for (int jt = 0; jt < C; ++jt) {
                        if (jt < n) {
                            const uint32_t word = lds32(stage + s * (C * 128u) + jt * 128u);
                            const uint2 d0 = decode8<0>(word, ll);  // strip row g
                            const uint2 d1 = decode8<1>(word, ll);  // strip row g + 8
                            uint32_t a[4], b[4];
                            bytes_to_half2(d0, a);
                            bytes_to_half2(d1, b);
#pragma unroll
                            for (int mb = 0; mb < MB; ++mb) {
                                mma_f16(acc[s][mb], a[0], b[0], a[1], b[1], xf[mb][jt][0], xf[mb][jt][1]);
                                mma_f16(acc[s][mb], a[2], b[2], a[3], b[3], xf[mb][jt][2], xf[mb][jt][3]);
                            }
                        }
                    }
                }
            }
            __syncwarp();  // every lane has read the stage: refill it
            if (icur.pos < icur.end) {
                issue(icur, iidx);
                icur.pos += chunk_tiles(icur);
                normalize(icur);
                ++iidx;
            }
            ccur.pos += n;
            normalize(ccur);
            ++cidx;
        }

        // ---- cross-warp reduction of this super-strip segment ----
#pragma unroll
        for (int s = 0; s < S; ++s)
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                acc_t *dst = red + warp * PSZ + (s * MB + mb) * 128 + lane * 4;
                *reinterpret_cast<int4 *>(dst) = *reinterpret_cast<int4 *>(acc[s][mb]);
            }
        __syncthreads();

        const bool full = (seg_a == ss_a) && (seg_b == ss_b);
        const int my_slot = seg_a > ss_a ? 0 : 1;
        acc_t *partials = reinterpret_cast<acc_t *>(p.partials);

        for (int o = tid; o < PSZ; o += kThreads) {
            acc_t tot = 0;
#pragma unroll
            for (int w = 0; w < NW; ++w) tot += red[w * PSZ + o];
            if (full) {
                store_out<Fam, S, MB>(p, ss, o, tot);
            } else {
                partials[(cta * 2 + my_slot) * PSZ + o] = tot;
            }
        }
        if (!full) __threadfence();
        __syncthreads();

        if (!full) {
            const long long c_lo = part_owner(T, G, ss_a), c_hi = part_owner(T, G, ss_b - 1);
            if (tid == 0) {
                const unsigned expected = static_cast<unsigned>(c_hi - c_lo + 1);
                const unsigned old = atomicAdd(p.tickets + ss, 1u);
                const int last = old == expected - 1;
                if (last) p.tickets[ss] = 0;  // ready for the next launch
                flags[1] = last;
            }
            __syncthreads();
            const bool last = flags[1] != 0;
            if (last) {
                __threadfence();
                for (int o = tid; o < PSZ; o += kThreads) {
                    acc_t tot = 0;
                    for (long long c = c_lo; c <= c_hi; ++c) {
                        const long long a_c = part_begin(T, G, c);
                        const int slot_c = a_c > ss_a ? 0 : 1;
                        tot += __ldcg(partials + (c * 2 + slot_c) * PSZ + o);
                    }
                    store_out<Fam, S, MB>(p, ss, o, tot);
                }
            }
            __syncthreads();  // flags[1] and red are reused by the next segment
        }
    }
}

template <class Fam, int S, int MB>
inline int launch_one(const StreamParams &p_in, int num_sms, bool pdl, cudaStream_t stream) {
    StreamParams p = p_in;
    using Plan = SmemPlan<S, MB>;
    p.dyn_smem_bytes = Plan::kDynBytes;
    auto kernel = stream_kernel<Fam, S, MB>;
    cudaError_t err =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Plan::kDynBytes));
    if (err != cudaSuccess) return err;
    const long long KT = p.K / 32, NS = p.N / 16, SS = (NS + S - 1) / S;
    const long long T = SS * KT;
    const unsigned grid = static_cast<unsigned>(T < num_sms ? T : num_sms);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kStreamWarps * 32);
    cfg.dynamicSmemBytes = Plan::kDynBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

inline int launch_stream(int family, const StreamParams &p, int num_sms, bool pdl, cudaStream_t stream) {
    if (family == 0) return DMM_ERR_UNSUPPORTED;  // the integer family runs on the tcgen05 kernel only
    if (p.M <= 8) return launch_one<FamF16, 4, 1>(p, num_sms, pdl, stream);
    return launch_one<FamF16, 2, 2>(p, num_sms, pdl, stream);
}

}  // namespace dmm
