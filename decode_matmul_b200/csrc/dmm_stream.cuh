// Streaming decode-matmul kernel (small-batch path, both families).
//
// One persistent CTA per SM.  The tiled code matrix is a linear stream of
// (N/16 strips) x (K/32 k-tiles) x 128 bytes; a work item is S strips x 4 k-tiles
// (a "super-strip" of 16*S output rows times 128 reduction indices, S*512 bytes of codes).
// Items are numbered super-strip-major and split evenly over the CTAs (stream-K), so every
// SM streams the same number of bytes whatever N and K are.
//
//   producer warp : one thread issues 1-D bulk copies (TMA) of item code bytes into a
//                   shared-memory ring, completion counted on an mbarrier per stage.
//   consumer warps: warp w takes items w, w+NW, ... of the CTA.  Per item and strip each
//                   lane reads 4 words (= 8 codes: rows g and g+8 of the strip, 4 k-tiles),
//                   decodes them with two table look-ups + XOR (dmm_common.cuh) and feeds
//                   legacy warp-level MMAs whose B operand is the activation fragment
//                   (batch along the MMA n dimension, 8 columns per group).
//   per super-strip: cross-warp reduction through shared memory, then either a direct
//                   store (the CTA covered the whole K range) or a partial written to the
//                   workspace; the last CTA to arrive (ticket counter) sums the partials in
//                   a fixed order and stores.  No CTA ever waits for another CTA.
//
// Fragment bookkeeping.  Lane l = 4g + t.  Word j of a lane holds the codes of strip rows
// g (low half) and g+8 (high half) for reduction indices k = 32*(4*kq + j) + 8*t + i.
// The MMA sums over "slots"; both operands use the same slot -> k map, so any map works:
//   fp16  m16n8k16: MMA 1 gets weights i = 0..3 (slots 2t,2t+1 | 2t+8,2t+9), MMA 2 i = 4..7.
//   int8  m16n8k32: slots 4t..4t+3 = i 0..3, slots 4t+16..4t+19 = i 4..7.
#pragma once
#include "dmm_common.cuh"
#include "dmm_launch.h"

namespace dmm {

struct FamI8 {
    using x_t = int8_t;
    using acc_t = int;
    static constexpr int kIsF16 = 0;
    static constexpr uint32_t kMaskExtra = 0x00u;
    static constexpr int kXRegs = 2;  // 8 int8 per k-tile per lane
};
struct FamF16 {
    using x_t = __half;
    using acc_t = float;
    static constexpr int kIsF16 = 1;
    static constexpr uint32_t kMaskExtra = 0x80u;
    static constexpr int kXRegs = 4;  // 8 halfs per k-tile per lane
};

constexpr int kRingStages = 32;

template <int S>
struct SmemPlan {
    static constexpr uint32_t kStageBytes = S * 512;
    static constexpr uint32_t kRingBytes = kRingStages * kStageBytes;
    static constexpr uint32_t kBarBytes = 1024;  // 2 * kRingStages mbarriers + flags
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
    if constexpr (Fam::kIsF16) {
        float *out = reinterpret_cast<float *>(p.out) + col * p.N + n;
        const float r = p.scale * v;
        *out = p.accumulate ? *out + r : r;
    } else {
        int *out = reinterpret_cast<int *>(p.out) + col * p.N + n;
        *out = p.accumulate ? *out + v : v;
    }
}

template <class Fam, int S, int MB, int NW>
__global__ void __launch_bounds__((NW + 1) * 32, 1) stream_kernel(const StreamParams p) {
    using acc_t = typename Fam::acc_t;
    constexpr int XR = Fam::kXRegs;
    constexpr int PSZ = S * MB * 128;  // accumulator values per super-strip
    constexpr uint32_t kStageBytes = SmemPlan<S>::kStageBytes;
    constexpr uint32_t kRedBytes = NW * PSZ * 4;
    constexpr uint32_t kPreBytes = SmemPlan<S>::kBarBytes + kRedBytes;
    constexpr int kConsumers = NW * 32;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t lut_addr = (base + kPreBytes + 0xFFFFu) & ~0xFFFFu;
    const uint32_t ring_addr = lut_addr + kLutBytes;
    const uint32_t bar_addr = base;          // full[kRingStages], empty[kRingStages]
    volatile int *flags = reinterpret_cast<volatile int *>(smem_raw + 2 * kRingStages * 8);  // [0]=failed [1]=last
    acc_t *red = reinterpret_cast<acc_t *>(smem_raw + SmemPlan<S>::kBarBytes);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;

    if (ring_addr + SmemPlan<S>::kRingBytes > base + p.dyn_smem_bytes) {  // uniform over the CTA
        if (tid == 0) raise_status(DMM_STATUS_BAD_SMEM);
        return;
    }

    const long long KT = p.K / 32;            // k-tiles per strip
    const long long KQ = (KT + 3) / 4;        // items per super-strip
    const long long NS = p.N / 16;            // strips
    const long long SS = (NS + S - 1) / S;    // super-strips
    const long long T = SS * KQ;
    const long long G = gridDim.x;
    const long long cta = blockIdx.x;
    const long long i0 = part_begin(T, G, cta), i1 = part_begin(T, G, cta + 1);
    const long long n_items = i1 - i0;

    if (tid == 0) {
        for (int s = 0; s < kRingStages; ++s) {
            mbar_init(bar_addr + 8u * s, 1);                  // full: producer's expect_tx arrival
            mbar_init(bar_addr + 8u * (kRingStages + s), 1);  // empty: one consumer lane
        }
        flags[0] = 0;
        flags[1] = 0;
        fence_mbar_init();
    }
    __syncthreads();
    grid_dep_launch();
    if (n_items <= 0) return;

    if (warp == NW) {
        // ------------------------------ producer ------------------------------
        if (lane == 0) {
            const uint64_t policy = policy_evict_first();
            const uint8_t *codes = reinterpret_cast<const uint8_t *>(p.codes);
            for (long long j = 0; j < n_items; ++j) {
                const long long i = i0 + j;
                const long long ss = i / KQ, kq = i - ss * KQ;
                const int slot = static_cast<int>(j % kRingStages);
                if (j >= kRingStages)
                    mbar_wait(bar_addr + 8u * (kRingStages + slot), static_cast<uint32_t>((j / kRingStages - 1) & 1), flags);
                const long long kt0 = 4 * kq;
                const uint32_t bytes = static_cast<uint32_t>((KT - kt0 < 4 ? KT - kt0 : 4) * 128);
                const int nstrips = static_cast<int>(NS - ss * S < S ? NS - ss * S : S);
                const uint32_t full = bar_addr + 8u * slot;
                mbar_arrive_expect_tx(full, bytes * nstrips);
                for (int s = 0; s < nstrips; ++s)
                    bulk_g2s(ring_addr + slot * kStageBytes + s * 512u,
                             codes + ((ss * S + s) * KT + kt0) * 128, bytes, full, policy);
            }
        }
        return;
    }

    // ---------------------------------- consumers ----------------------------------
    const bool bad = lut_fill(lut_addr, p.cb, p.cb_is_f16, p.sign_convention, Fam::kMaskExtra, tid, kConsumers);
    if (bad) raise_status(DMM_STATUS_BAD_CODEBOOK);
    named_barrier(1, kConsumers);
    const LutLane ll = lut_lane(lut_addr, lane);

    grid_dep_wait();  // activations, out (accumulate), workspace: only after the previous kernel

    const int g = lane >> 2, t = lane & 3;
    const typename Fam::x_t *x = reinterpret_cast<const typename Fam::x_t *>(p.x);

    long long j_base = 0;
    const long long ss_first = i0 / KQ, ss_last = (i1 - 1) / KQ;
    for (long long ss = ss_first; ss <= ss_last; ++ss) {
        const long long seg_a = i0 > ss * KQ ? i0 : ss * KQ;
        const long long seg_b = i1 < (ss + 1) * KQ ? i1 : (ss + 1) * KQ;
        const long long len = seg_b - seg_a;
        const int nstrips = static_cast<int>(NS - ss * S < S ? NS - ss * S : S);

        acc_t acc[S][MB][4];
#pragma unroll
        for (int s = 0; s < S; ++s)
#pragma unroll
            for (int mb = 0; mb < MB; ++mb)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[s][mb][c] = 0;

        long long j = j_base + ((warp - j_base % NW) + NW) % NW;
        for (; j < j_base + len; j += NW) {
            const long long kq = (seg_a - ss * KQ) + (j - j_base);
            const int slot = static_cast<int>(j % kRingStages);
            const int ktv = static_cast<int>(KT - 4 * kq < 4 ? KT - 4 * kq : 4);  // valid k-tiles

            // activation fragments: xf[mb][jt][r], 8 consecutive k per (lane, k-tile)
            uint32_t xf[MB][4][XR];
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                const long long col = mb * 8 + g;
#pragma unroll
                for (int jt = 0; jt < 4; ++jt) {
#pragma unroll
                    for (int r = 0; r < XR; ++r) xf[mb][jt][r] = 0;
                    if (col < p.M && jt < ktv) {
                        const typename Fam::x_t *src = x + col * p.K + 32 * (4 * kq + jt) + 8 * t;
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

            mbar_wait(bar_addr + 8u * slot, static_cast<uint32_t>((j / kRingStages) & 1), flags);
            const uint32_t stage = ring_addr + slot * kStageBytes + lane * 4u;

#pragma unroll
            for (int s = 0; s < S; ++s) {
                if (s < nstrips) {
#pragma unroll
                    for (int jt = 0; jt < 4; ++jt) {
                        if (jt < ktv) {
                            const uint32_t word = lds32(stage + s * 512u + jt * 128u);
                            const uint2 d0 = decode8<0>(word, ll);  // strip row g
                            const uint2 d1 = decode8<1>(word, ll);  // strip row g + 8
                            if constexpr (Fam::kIsF16) {
                                uint32_t a[4], b[4];
                                bytes_to_half2(d0, a);
                                bytes_to_half2(d1, b);
#pragma unroll
                                for (int mb = 0; mb < MB; ++mb) {
                                    mma_f16(acc[s][mb], a[0], b[0], a[1], b[1], xf[mb][jt][0], xf[mb][jt][1]);
                                    mma_f16(acc[s][mb], a[2], b[2], a[3], b[3], xf[mb][jt][2], xf[mb][jt][3]);
                                }
                            } else {
#pragma unroll
                                for (int mb = 0; mb < MB; ++mb)
                                    mma_s8(acc[s][mb], d0.x, d1.x, d0.y, d1.y, xf[mb][jt][0], xf[mb][jt][1]);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_addr + 8u * (kRingStages + slot));
        }
        j_base += len;

        // ---- cross-warp reduction of this super-strip segment ----
#pragma unroll
        for (int s = 0; s < S; ++s)
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                acc_t *dst = red + warp * PSZ + (s * MB + mb) * 128 + lane * 4;
                *reinterpret_cast<int4 *>(dst) = *reinterpret_cast<int4 *>(acc[s][mb]);
            }
        named_barrier(1, kConsumers);

        const bool full = (seg_a == ss * KQ) && (seg_b == (ss + 1) * KQ);
        const int my_slot = seg_a > ss * KQ ? 0 : 1;
        acc_t *partials = reinterpret_cast<acc_t *>(p.partials);

        for (int o = tid; o < PSZ; o += kConsumers) {
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
        named_barrier(1, kConsumers);

        if (!full) {
            const long long c_lo = part_owner(T, G, ss * KQ), c_hi = part_owner(T, G, (ss + 1) * KQ - 1);
            if (tid == 0) {
                const unsigned expected = static_cast<unsigned>(c_hi - c_lo + 1);
                const unsigned old = atomicAdd(p.tickets + ss, 1u);
                const int last = old == expected - 1;
                if (last) p.tickets[ss] = 0;  // ready for the next launch
                flags[1] = last;
            }
            named_barrier(1, kConsumers);
            const bool last = flags[1] != 0;
            if (last) {
                __threadfence();
                for (int o = tid; o < PSZ; o += kConsumers) {
                    acc_t tot = 0;
                    for (long long c = c_lo; c <= c_hi; ++c) {
                        const long long a_c = part_begin(T, G, c);
                        const int slot_c = a_c > ss * KQ ? 0 : 1;
                        tot += __ldcg(partials + (c * 2 + slot_c) * PSZ + o);
                    }
                    store_out<Fam, S, MB>(p, ss, o, tot);
                }
            }
            named_barrier(1, kConsumers);  // flags[1] and red are reused by the next segment
        }
    }
}


template <class Fam, int S, int MB, int NW>
inline int launch_one(const StreamParams &p_in, int num_sms, bool pdl, cudaStream_t stream) {
    StreamParams p = p_in;
    constexpr unsigned kPre = SmemPlan<S>::kBarBytes + NW * S * MB * 128 * 4;
    // table needs a 64 KiB-aligned address: reserve worst-case slack
    constexpr unsigned kDyn = kPre + 0xFFFFu + kLutBytes + SmemPlan<S>::kRingBytes;
    static_assert(kDyn <= 232448 - 1024, "shared memory plan exceeds the per-CTA limit");
    p.dyn_smem_bytes = kDyn;
    auto kernel = stream_kernel<Fam, S, MB, NW>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kDyn));
    if (err != cudaSuccess) return err;
    const long long KT = p.K / 32, KQ = (KT + 3) / 4, NS = p.N / 16, SS = (NS + S - 1) / S;
    const long long T = SS * KQ;
    const unsigned grid = static_cast<unsigned>(T < num_sms ? T : num_sms);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3((NW + 1) * 32);
    cfg.dynamicSmemBytes = kDyn;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

inline int launch_stream(int family, const StreamParams &p, int num_sms, bool pdl, cudaStream_t stream) {
    constexpr int NW = 16;
    if (family == 0) {
        if (p.M <= 8) return launch_one<FamI8, 4, 1, NW>(p, num_sms, pdl, stream);
        return launch_one<FamI8, 2, 2, NW>(p, num_sms, pdl, stream);
    }
    if (p.M <= 8) return launch_one<FamF16, 4, 1, NW>(p, num_sms, pdl, stream);
    return launch_one<FamF16, 2, 2, NW>(p, num_sms, pdl, stream);
}

}  // namespace dmm
