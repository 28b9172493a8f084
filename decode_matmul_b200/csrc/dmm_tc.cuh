// Second tcgen05 decode-matmul kernel for the fp6/fp8-operand policy (fp16 family) and the int8 policy,
// one launch per product.  Same data path as the kernel of dmm_umma.cuh (read that header first) with a
// different division of labour around it: one TMA producer per decoder group, activations staged in
// fixed "rounds" so that an MMA issuer finds its operands by increments, leaner issuer loops.  The
// library uses it for 17 to 32 batch rows, where the single in-order issuer pair of the first kernel
// is the limit.
//
// Decoded weights are the A operand of tcgen05.mma and live only in tensor memory: a decoder
// thread owns two output rows, decodes their codes in registers (two table look-ups and two XORs
// per code) and writes them with tcgen05.st.  The activations are the B operand, staged in shared
// memory in the canonical no-swizzle K-major layout; accumulators live in TMEM.
//
// Work decomposition.  A super-tile is 16 strips = 256 output rows = two M=128 MMA tiles (tile 0:
// strip rows 0..7, tile 1: strip rows 8..15, because one 16-byte piece of the tiled code stream
// holds the codes of rows g and g+8 and one thread decodes both).  A "tile" of work is
// (super-tile, k-tile): 2 KiB of codes.  Tiles are numbered super-tile-major and split evenly and
// contiguously over the CTAs (stream-K); the part of a super-tile a CTA owns is a segment.  The
// CTA's tiles are cut into chunks of C = 4 k-tiles (one TMA box, 8 KiB), numbered through all
// segments; chunk number mod 4 is the decoder group that handles it.
//
// Warp roles (28 warps):
//   0..15   decoders, four groups of four warps.  Warp wq of a group owns TMEM lanes 32wq..32wq+31
//           = strips 4wq..4wq+3.  Per step (G = 2 k-tiles) it decodes 16 codes per lane into one of
//           NA group buffers in TMEM and signals the group's MMA issuer.  The decoders also build
//           the look-up table at the start; groups 0 and 1 run the epilogue of MMA tile 0 and 1.
//   16..19  MMA issuers (converged warps, one elected lane issues).  Issuer `me` serves the chunks
//           whose number is me mod NACC and owns accumulator set `me`; with fewer than four sets
//           the two MMA tiles of a chunk are issued by two warps (so that each accumulator still
//           has exactly one issuer and the summation order is fixed).
//   20..23  activation loaders.  The activations of the CTA's k-tile sequence are staged round by
//           round: a round is NACC consecutive chunks (one per issuer), kept in one of NE round buffers
//           (3 at the largest round size, up to 8 for small batches); loader w owns the buffers b with
//           b mod 4 = w and fills their rounds.  Slot (chunk j of the round, k-tile i) sits at a fixed offset, so an issuer finds its operands without any search: it uses
//           exactly one chunk of every round, in order.  The loaders are the only warps that wait
//           for the previous kernel of the stream (programmatic dependent launch).
//   24..27  TMA producers, one thread per decoder group: they stream that group's code chunks
//           into the group's own ring, one tiled bulk-tensor load per chunk.
// Every wait is a bounded mbarrier wait (mbar_wait); nothing spins on another CTA.
#pragma once
#include "dmm_umma.cuh"

namespace dmm {

constexpr int kTcDecWarps = 16, kTcMmaWarp = 16, kTcMmaWarps = 4, kTcLoadWarp = 20, kTcLoadWarps = 4, kTcTmaWarp = 24,
              kTcTmaWarps = 4;
constexpr int kTcThreads = (kTcDecWarps + kTcMmaWarps + kTcLoadWarps + kTcTmaWarps) * 32;
constexpr uint32_t kTcBarBytes = 2048;
constexpr uint32_t kTcRoundBytes = 16384;  // activation planes of one round (NACC chunks of C k-tiles), at most
constexpr int kTcRounds = 3;               // round buffers at the largest round size
constexpr int kTcMaxRounds = 8;            // and at most this many when the rounds are small (few batch rows)

template <class Pol, int NMMA>
struct TcPlan {
    static_assert(Pol::kIsF8, "fp6/fp8 and int8 operand policies only");
    static constexpr int kG = 2, kNA = 2, kC = 4, kRing = 3;
    // accumulator sets = issuers that share the work: one per decoder group while the TMEM holds them
    static constexpr int kNAcc = NMMA <= 32 ? 4 : (NMMA <= 64 ? 2 : 1);
    static constexpr int kLogNAcc = kNAcc == 4 ? 2 : (kNAcc == 2 ? 1 : 0);
    static constexpr int kTileParts = kNAcc <= 2 ? 2 : 1;            // issuer warps per accumulator set
    static constexpr uint32_t kDCols = 2 * kNAcc * NMMA;             // TMEM: accumulators first
    static constexpr uint32_t kBufCols = 2 * kG * 8;                 // one group buffer: [tile][k-tile][8 columns]
    static constexpr uint32_t kACols = 4 * kNA * kBufCols;
    static_assert(kDCols + kACols <= 512, "TMEM plan exceeds 512 columns");
    static constexpr int kSlots = 4 * kNA;
    static constexpr int kNB = Pol::out_cols(NMMA);                  // batch columns per launch
    static constexpr uint32_t kXBytes = kTcRounds * kTcRoundBytes + 256;
    static constexpr uint32_t kPreBytes = kTcBarBytes + kXBytes;
    static constexpr uint32_t kSlotBytes = 16 * kC * 128;            // ring slot: 16 strips x C k-tiles (one TMA box)
    static constexpr uint32_t kRingBytes = 4 * kRing * kSlotBytes;   // one ring per decoder group
    static constexpr uint32_t kDynBytes = 0x10000u - 0x400u + kLutBytes + kRingBytes;
    static constexpr int kPartial = 2 * kNB * 128;                   // output values per segment
    static_assert(kPreBytes <= 0x10000u - 0x400u, "activation rounds do not fit below the table");
    static_assert(kDynBytes <= 232448u, "shared memory plan exceeds the per-CTA limit");
    // barrier indices
    static constexpr int kBarCode = 0;                               // [4][kRing] TMA completion
    static constexpr int kBarEmpty = kBarCode + 4 * kRing;           // [4][kRing] the group's 4 warps are done
    static constexpr int kBarFull = kBarEmpty + 4 * kRing;           // [kSlots] decoder warps
    static constexpr int kBarFree = kBarFull + kSlots;               // [kSlots] tcgen05.commit
    static constexpr int kBarXReady = kBarFree + kSlots;             // [kTcMaxRounds] loader
    static constexpr int kBarXFree = kBarXReady + kTcMaxRounds;      // [kTcMaxRounds] every issuer (commit)
    static constexpr int kBarDReady = kBarXFree + kTcMaxRounds;
    static constexpr int kBarDFree = kBarDReady + 1;
    static constexpr int kBarCount = kBarDFree + 1;
    static_assert(kBarCount * 8 + 64 <= kTcBarBytes, "barrier block too small");
};

// Bytes of the activation operand of one k-tile: fp8 planes [k-half][plane][row][16 B] with the rows
// of a plane packed densely (M rows, up to 8) or padded to 16 / 32 rows for the 64- and 128-column
// variants; int8: [k-half][row < NMMA][16 B].
template <class Pol, int NMMA>
__host__ __device__ inline uint32_t tc_tile_bytes(int M) {
    return plane_tile_bytes<NMMA, Pol::kIsInt != 0>(M);
}

// Bytes of one activation round (one chunk per issuer: NACC chunks of C k-tiles) and the number of round
// buffers that fit the activation area: 3 at the largest round, up to 8 when the batch is small, so that
// the loaders work several rounds (microseconds) ahead of the MMAs.
template <class Pol, int NMMA>
__host__ __device__ inline uint32_t tc_round_bytes(int M) {
    return static_cast<uint32_t>(TcPlan<Pol, NMMA>::kNAcc * TcPlan<Pol, NMMA>::kC) * tc_tile_bytes<Pol, NMMA>(M);
}
template <class Pol, int NMMA>
__host__ __device__ inline int tc_rounds(int M) {
    const int fit = static_cast<int>((kTcRounds * kTcRoundBytes) / tc_round_bytes<Pol, NMMA>(M));
    return fit < kTcMaxRounds ? fit : kTcMaxRounds;
}

struct TcArgs {
    UmmaParams p;
    CUtensorMap map;
};

template <class Pol, int NMMA, bool kTp>
__global__ void __launch_bounds__(kTcThreads, 1) dmm_kernel(const __grid_constant__ TcArgs args) {
    using Plan = TcPlan<Pol, NMMA>;
    constexpr int C = Plan::kC, G = Plan::kG, NA = Plan::kNA, RING = Plan::kRing, NACC = Plan::kNAcc, NB = Plan::kNB;
    constexpr int TP = Plan::kTileParts, LOGNACC = Plan::kLogNAcc;
    constexpr bool kInt = Pol::kIsInt != 0;
    const UmmaParams &p = args.p;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t lut_addr = (base + Plan::kPreBytes + 0xFFFFu) & ~0xFFFFu;
    const uint32_t ring_addr = lut_addr + kLutBytes;
    const uint32_t x_addr = base + kTcBarBytes;
    volatile int *flags = reinterpret_cast<volatile int *>(smem_raw + Plan::kBarCount * 8);  // [0]=failed [1]=last [2]=2
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_raw + Plan::kBarCount * 8 + 16);
    auto bar = [&](int i) -> uint32_t { return base + 8u * static_cast<uint32_t>(i); };

    // the warp index through a shuffle: the compiler then knows it is the same in every lane and
    // keeps what derives from it (roles, descriptors, TMEM addresses) in uniform registers
    const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
    // the codebook is static data: fetch it first (fp16 table; the int64 table is read in lut_fill)
    const uint4 cb_pre = kInt ? make_uint4(0, 0, 0, 0) : lut_prefetch(p.cb, tid);

    if (ring_addr + Plan::kRingBytes > base + p.dyn_smem_bytes) {  // uniform over the grid
        if (tid == 0) raise_status(DMM_STATUS_BAD_SMEM);
        return;
    }

    // This CTA's tiles [i0, i1) of the (super-tile, k-tile) sequence and the segments they span.
    const int cta = blockIdx.x;
    const int KT = static_cast<int>(p.K / 32);
    const int i0 = part32_begin(p.part, cta), i1 = part32_begin(p.part, cta + 1);
    const int ss_first = i0 / KT, ss_last = i1 > i0 ? (i1 - 1) / KT : ss_first - 1;
    auto seg_kt0 = [&](int ss) -> int {
        const int a = ss * KT;
        return i0 > a ? i0 - a : 0;
    };
    auto seg_len = [&](int ss) -> int {
        const int a = ss * KT;
        const int lo = i0 > a ? i0 : a, hi = i1 < a + KT ? i1 : a + KT;
        return hi - lo;
    };
    auto seg_chunks = [&](int ss) -> int { return (seg_len(ss) + C - 1) / C; };

    // ---- set-up ----
    // The decoder warps build the look-up table straight away; the other warps initialise the
    // barriers and allocate TMEM meanwhile and then go on (the code stream starts flowing while the
    // table is still being built).  The decoders join through barrier 4, on which the others only arrive.
    constexpr int kOtherThreads = kTcThreads - kTcDecWarps * 32;
    bool bad_cb = false;
    if (warp < kTcDecWarps) {
        bad_cb = lut_fill(lut_addr, p.cb, kInt ? 0 : 1, p.sign_convention, Pol::kFmt, tid, kTcDecWarps * 32, !kInt,
                          kInt ? nullptr : &cb_pre);
        named_barrier(4, kTcThreads);
    } else {
        const int ot = tid - kTcDecWarps * 32;  // 0 .. kOtherThreads-1
        const int bt = ot - kTcMmaWarps * 32;   // loader and TMA warps initialise the barriers
        if (bt >= 0 && bt < Plan::kBarCount) {
            uint32_t count = 1;                                                    // TMA, loader, tcgen05.commit
            if (bt >= Plan::kBarEmpty && bt < Plan::kBarFull) count = 4;           // the group's decoder warps
            if (bt >= Plan::kBarFull && bt < Plan::kBarFree) count = 4;
            if (bt >= Plan::kBarFree && bt < Plan::kBarXReady) count = TP;         // every issuer of the slot
            if (bt >= Plan::kBarXFree && bt < Plan::kBarDReady) count = NACC * TP;
            if (bt == Plan::kBarDReady) count = NACC * TP;
            if (bt == Plan::kBarDFree) count = 8;
            mbar_init(bar(bt), count);
            if (bt == 0) {
                flags[0] = 0;
                flags[1] = 0;
                flags[2] = 2;
            }
            fence_mbar_init();
        }
        if (warp == kTcMmaWarp) tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), 512);
        fence_async_smem();
        tc_fence_before();
        named_barrier(3, kOtherThreads);
        named_barrier_arrive(4, kTcThreads);
    }
    tc_fence_after();
    const uint32_t tmem = __shfl_sync(0xffffffffu, *tmem_slot, 0);
    grid_dep_launch();

    if (warp < kTcDecWarps) {
        // =============================== decoders ===============================
        // Nothing here reads what an earlier kernel of the stream wrote (codes and codebook are
        // static), so the decoders never wait for it: they decode ahead into TMEM while the
        // previous kernel drains; the activation loaders are the ones that wait.
        const int q = warp >> 2, wq = warp & 3;
        const uint32_t gring = ring_addr + static_cast<uint32_t>(q) * (RING * Plan::kSlotBytes);  // ring of group q
        if (bad_cb) raise_status(DMM_STATUS_BAD_CODEBOOK);
        LutLane ll = lut_lane(lut_addr, lane, !kInt);
        ll.two = static_cast<uint32_t>(flags[2]);
        const uint32_t tlane = tmem + (static_cast<uint32_t>(wq * 32) << 16);
        const uint32_t abase = tlane + Plan::kDCols + static_cast<uint32_t>(q * NA) * Plan::kBufCols;
        // lane's place in a ring slot [16 strips][C k-tiles][128 B]: strip 4*wq + lane/8, piece lane%8
        const uint32_t lane_off = (wq * 4 + (lane >> 3)) * (C * 128) + (lane & 7) * 16;
        int slot = 0;            // ring slot of the next chunk, and the phase parity of its barriers
        uint32_t cpar = 0;
        int buf = 0;             // group buffer of the next step
        uint32_t fpar = 1;       // parity to wait for on its Free barrier (the first NA steps find it free)
        int segidx = 0, ebase = 0;  // segments and chunks of this CTA so far
        for (int ss = ss_first; ss <= ss_last; ebase += seg_chunks(ss), ++ss, ++segidx) {
            const int len = seg_len(ss);
            const int nchunks_ss = (len + C - 1) / C;
            for (int c = (q - ebase) & 3; c < nchunks_ss; c += 4) {
                const int n = len - c * C < C ? len - c * C : C;  // k-tiles in this chunk
                mbar_wait(bar(Plan::kBarCode + q * RING + slot), cpar, flags);
                const uint32_t src = gring + slot * Plan::kSlotBytes + lane_off;
#pragma unroll 1
                for (int g0 = 0; g0 < n; g0 += G) {
                    const int sl = q * NA + buf;
                    mbar_wait(bar(Plan::kBarFree + sl), fpar, flags);
                    tc_fence_after();
                    const uint32_t acol = abase + static_cast<uint32_t>(buf) * Plan::kBufCols;
                    // group buffer columns: [tile][k-tile][8]; two k-tiles -> one x16 store per tile
                    uint32_t r0[8 * G], r1[8 * G];
#pragma unroll
                    for (int i = 0; i < G; ++i) {
                        uint4 cw = make_uint4(0, 0, 0, 0);
                        if (g0 + i < n) cw = lds128(src + (g0 + i) * 128);
                        const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            uint2 d0, d1;
                            if constexpr (kInt) {
                                d0 = decode8<0>(w[t], ll);
                                d1 = decode8<1>(w[t], ll);
                            } else {
                                d0 = decode8_fp6<0>(w[t], ll);
                                d1 = decode8_fp6<1>(w[t], ll);
                            }
                            r0[8 * i + 2 * t] = d0.x; r0[8 * i + 2 * t + 1] = d0.y;
                            r1[8 * i + 2 * t] = d1.x; r1[8 * i + 2 * t + 1] = d1.y;
                        }
                    }
                    static_assert(G == 2, "two k-tiles per step: one x16 store per MMA tile");
                    tmem_st16(acol, reinterpret_cast<const uint32_t(&)[16]>(r0));
                    tmem_st16(acol + G * 8, reinterpret_cast<const uint32_t(&)[16]>(r1));
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(Plan::kBarFull + sl));
                    if (++buf == NA) {
                        buf = 0;
                        fpar ^= 1u;
                    }
                }
                __syncwarp();  // every lane has read the slot: hand it back to the TMA producer
                if (lane == 0) mbar_arrive(bar(Plan::kBarEmpty + q * RING + slot));
                if (++slot == RING) {
                    slot = 0;
                    cpar ^= 1u;
                }
            }

            if (q < 2) {
                // ---------------- epilogue of MMA tile q of this segment ----------------
                // accumulator set a was written in this segment iff one of its chunks is a mod NACC
                uint32_t used = 0;
                for (int cc = 0; cc < nchunks_ss && cc < NACC; ++cc) used |= 1u << ((ebase + cc) % NACC);
                mbar_wait(bar(Plan::kBarDReady), static_cast<uint32_t>(segidx & 1), flags);
                tc_fence_after();
                // the accumulators are fp32, or int32 for the integer family (exact, no scale)
                using Acc = typename AccType<kInt>::type;
                Acc v[NB];
#pragma unroll
                for (int b = 0; b < NB; ++b) v[b] = Acc(0);
                Acc *const out_acc = reinterpret_cast<Acc *>(p.out);
                Acc *const partials_acc = reinterpret_cast<Acc *>(p.partials);
                if (!kInt && p.M == 1) {
                    // batch 1: only column 8 * plane of every accumulator carries data; fetch those
                    // sixteen words with one wait instead of whole accumulators one after the other
                    uint32_t r[16];
#pragma unroll
                    for (int a = 0; a < 4; ++a) {
#pragma unroll
                        for (int pl = 0; pl < 4; ++pl) {
                            r[a * 4 + pl] = 0u;
                            if (a < NACC && ((used >> a) & 1u))
                                r[a * 4 + pl] = tmem_ld1(tlane + static_cast<uint32_t>((q * NACC + a) * NMMA + 8 * pl));
                        }
                    }
                    tmem_wait_ld(r);
#pragma unroll
                    for (int e = 0; e < 16; ++e) v[0] += acc_from_bits<Acc>(r[e]);
                } else {
#pragma unroll
                    for (int a = 0; a < NACC; ++a) {
                        if ((used >> a) & 1u) {
#pragma unroll
                            for (int b0 = 0; b0 < NMMA; b0 += 16) {
                                uint32_t r[16];
                                tmem_ld16(tlane + static_cast<uint32_t>((q * NACC + a) * NMMA + b0), r);
                                tmem_wait_ld(r);
                                // fp8 planes: column 8*plane + b (or 16*plane + b, 32*plane + b); int8: column b
#pragma unroll
                                for (int e = 0; e < 16; ++e) v[(b0 + e) % NB] += acc_from_bits<Acc>(r[e]);
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(Plan::kBarDFree));

                const int ss_a = ss * KT;
                const bool full = len == KT;
                const int my_slot = seg_kt0(ss) > 0 ? 0 : 1;
                const int trow = wq * 32 + lane;  // TMEM lane = row of the MMA tile
                const long long n = (static_cast<long long>(ss) * 16 + wq * 4 + (lane >> 3)) * 16 + 8 * q + (lane & 7);
                const int ptid = q * 128 + trow;
                if (p.atomic_reduce) {
                    if (n < p.N) {
                        if (kTp && p.n_peers > 0) {
                            // the same element on every rank: system-scope adds over NVLink peer memory
                            for (int r = 0; r < p.n_peers; ++r) {
#pragma unroll
                                for (int b = 0; b < NB; ++b)
                                    if (b < p.M) atomicAdd_system(reinterpret_cast<Acc *>(p.peer_out[r]) + b * p.N + n, acc_scaled(p.scale, v[b]));
                            }
                        } else {
#pragma unroll
                            for (int b = 0; b < NB; ++b)
                                if (b < p.M) atomicAdd(out_acc + b * p.N + n, acc_scaled(p.scale, v[b]));
                        }
                    }
                } else if (full) {
                    if (n < p.N) {
#pragma unroll
                        for (int b = 0; b < NB; ++b)
                            if (b < p.M) {
                                Acc *o = out_acc + b * p.N + n;
                                const Acc r = acc_scaled(p.scale, v[b]);
                                *o = p.accumulate ? *o + r : r;
                            }
                    }
                } else {
                    Acc *mine = partials_acc + static_cast<long long>(cta * 2 + my_slot) * Plan::kPartial + q * NB * 128 + trow;
#pragma unroll
                    for (int b = 0; b < NB; ++b)
                        if (b < p.M) mine[b * 128] = v[b];
                    __threadfence();
                    named_barrier(2, 256);
                    const int c_lo = part32_owner(p.part, ss_a), c_hi = part32_owner(p.part, ss_a + KT - 1);
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
                            const int ncta = c_hi - c_lo + 1;
#pragma unroll
                            for (int b = 0; b < NB; ++b)
                                if (b < p.M) {
                                    // fixed summation order; eight loads in flight at a time
                                    Acc tot = Acc(0);
                                    for (int c0 = 0; c0 < ncta; c0 += 8) {
                                        Acc part[8];
#pragma unroll
                                        for (int e = 0; e < 8; ++e) {
                                            part[e] = Acc(0);
                                            if (c0 + e < ncta) {
                                                const int c = c_lo + c0 + e;
                                                const int slot_c = part32_begin(p.part, c) > ss_a ? 0 : 1;
                                                part[e] = __ldcg(partials_acc + static_cast<long long>(c * 2 + slot_c) * Plan::kPartial +
                                                                 (q * NB + b) * 128 + trow);
                                            }
                                        }
#pragma unroll
                                        for (int e = 0; e < 8; ++e) tot += part[e];
                                    }
                                    Acc *o = out_acc + b * p.N + n;
                                    const Acc r = acc_scaled(p.scale, tot);
                                    *o = p.accumulate ? *o + r : r;
                                }
                        }
                    }
                    named_barrier(2, 256);  // flags[1] is reused by the next segment
                }
            }
        }
    } else if (warp < kTcMmaWarp + kTcMmaWarps) {
        // =============================== MMA issuers ===============================
        // Issuer (me, tp) takes the chunks whose CTA-wide number is me mod NACC -- exactly one chunk of
        // every activation round, in order -- and owns accumulator set `me` (of MMA tile tp when the
        // tiles are split).  The warp runs converged; one elected lane issues.  Everything an MMA
        // needs is an increment of something kept from the step before.
        const int wi = warp - kTcMmaWarp;
        const int me = wi % NACC, tp = wi / NACC;
        if (wi < NACC * TP) {
            const bool leader = elect_one();
            // instruction descriptor: D fp32 (1) or int32 (2) at bit 4; A / B formats at bits 7 / 10
            // (f8f6f4: E2M3 = 3, E5M2 = 1; i8: signed = 1); N >> 3 at 17; M >> 4 at 24
            const uint32_t idesc = kInt ? ((2u << 4) | (1u << 7) | (1u << 10) | ((NMMA >> 3) << 17) | ((128u >> 4) << 24))
                                        : ((1u << 4) | (3u << 7) | (1u << 10) | ((NMMA >> 3) << 17) | ((128u >> 4) << 24));
            const uint32_t tile_b = tc_tile_bytes<Pol, NMMA>(static_cast<int>(p.M));
            // fp8: a plane is one 8-row core matrix (rows past the batch overlap the next plane and land
            // in unused columns) or, for the padded layouts, two or four of them
            const uint64_t xdesc0 = smem_desc(x_addr, tile_b / 2, (NMMA > 32 || kInt) ? 128u : tile_b / 8);
            const uint32_t xdesc_hi = static_cast<uint32_t>(xdesc0 >> 32);
            const uint32_t tile16 = tile_b >> 4;
            // A round holds one chunk of every issuer: chunk number ci sits at slot ci mod NACC, mine is slot
            // `me`.  Operand of its k-tile 0 in round buffer 0; the NE round buffers follow one another:
            const int NE = tc_rounds<Pol, NMMA>(static_cast<int>(p.M));
            const uint32_t x_first = static_cast<uint32_t>(xdesc0) + static_cast<uint32_t>(me * C) * tile16;
            const uint32_t x_step = static_cast<uint32_t>(NACC * C) * tile16;  // one round buffer
            uint32_t x_cur = x_first;
            int rb = 0;              // round buffer of my next chunk
            uint32_t xpar = 0;       // parity of its XReady phase
            // accumulator(s): MMA tile t of set me sits at column (t * NACC + me) * NMMA
            const uint32_t d_col0 = tmem + static_cast<uint32_t>(((TP == 2 ? tp : 0) * NACC + me) * NMMA);
            const uint32_t a_tile = TP == 2 ? static_cast<uint32_t>(tp * G * 8) : 0u;  // my MMA tile inside a group buffer
            // per decoder group I serve: next group buffer and the parity of its Full phase
            // (NACC == 4: one group; 2: groups me, me + 2; 1: all four)
            uint32_t sbuf = 0, spar = 0;  // bit q: buffer index (NA == 2) and parity of group q
            static_assert(NA == 2, "buffer index kept as one bit per group");
            int segidx = 0, cbase = 0;
            for (int ss = ss_first; ss <= ss_last; cbase += seg_chunks(ss), ++ss, ++segidx) {
                const int len = seg_len(ss);
                const int nchunks = (len + C - 1) / C;
                if (segidx > 0) {
                    mbar_wait(bar(Plan::kBarDFree), static_cast<uint32_t>((segidx - 1) & 1), flags);
                    tc_fence_after();
                }
                uint32_t acc = 0u;  // the accumulators hold nothing of this segment yet
                for (int c = (me - cbase) & (NACC - 1); c < nchunks; c += NACC) {
                    const int q = (cbase + c) & 3;
                    const int n = len - c * C < C ? len - c * C : C;
                    mbar_wait(bar(Plan::kBarXReady + rb), xpar, flags);
#pragma unroll 1
                    for (int g0 = 0; g0 < n; g0 += G) {
                        const uint32_t b = (sbuf >> q) & 1u;
                        const int sl = q * NA + static_cast<int>(b);
                        mbar_wait(bar(Plan::kBarFull + sl), (spar >> q) & 1u, flags);
                        tc_fence_after();
                        if (leader) {
                            const uint32_t a_col = tmem + Plan::kDCols + static_cast<uint32_t>(sl) * Plan::kBufCols + a_tile;
                            const uint32_t xlo = x_cur + static_cast<uint32_t>(g0) * tile16;
#pragma unroll
                            for (int i = 0; i < G; ++i) {
                                if (g0 + i < n) {
                                    if constexpr (TP == 1) {
                                        mma_ts_f8_lh<kInt>(d_col0, a_col + i * 8, xlo + i * tile16, xdesc_hi, idesc, acc);
                                        mma_ts_f8_lh<kInt>(d_col0 + NACC * NMMA, a_col + (G + i) * 8, xlo + i * tile16, xdesc_hi, idesc, acc);
                                    } else {
                                        mma_ts_f8_lh<kInt>(d_col0, a_col + i * 8, xlo + i * tile16, xdesc_hi, idesc, acc);
                                    }
                                    acc = 1u;
                                }
                            }
                            tc_commit(bar(Plan::kBarFree + sl));
                        }
                        acc = 1u;
                        sbuf ^= 1u << q;
                        if (b == 1u) spar ^= 1u << q;
                    }
                    // this round's operands are no longer needed once the MMAs above have completed
                    if (leader) tc_commit(bar(Plan::kBarXFree + rb));
                    x_cur += x_step;
                    if (++rb == NE) {
                        rb = 0;
                        xpar ^= 1u;
                        x_cur = x_first;
                    }
                }
                if (leader) tc_commit(bar(Plan::kBarDReady));
            }
        }
    } else if (warp >= kTcTmaWarp) {
        // =============================== TMA producers ===============================
        // One thread per decoder group streams that group's code chunks, one tiled load (16 strips x
        // C k-tiles) per chunk into the group's own ring.  Always the full box: k-tiles past the
        // segment are not used, strips past N read as zero.
        const int q = warp - kTcTmaWarp;
        if (lane == 0) {
            const uint64_t policy = policy_evict_first();
            uint32_t n_q = 0;      // chunks issued for this group
            int slot = 0;
            uint32_t par = 1;      // parity of the Empty phase that frees `slot` (first pass: nothing to wait for)
            int cbase = 0;
            for (int ss = ss_first; ss <= ss_last; cbase += seg_chunks(ss), ++ss) {
                const int nchunks = seg_chunks(ss), kt0 = seg_kt0(ss);
                for (int c = (q - cbase) & 3; c < nchunks; c += 4) {
                    if (n_q >= RING) mbar_wait(bar(Plan::kBarEmpty + q * RING + slot), par, flags);
                    const uint32_t b = bar(Plan::kBarCode + q * RING + slot);
                    mbar_arrive_expect_tx(b, Plan::kSlotBytes);
                    tma_load_2d(ring_addr + (q * RING + slot) * Plan::kSlotBytes, &args.map, (kt0 + c * C) * 32, ss * 16, b, policy);
                    ++n_q;
                    if (++slot == RING) {
                        slot = 0;
                        par ^= 1u;
                    }
                }
            }
            prefetch_next_codes(p, cta, q, 4, 4 * RING * C);
            if (flags[0]) {
                // A wait gave up somewhere: loads may still be in flight.  Give the last load of
                // every ring slot a bounded chance to land before the CTA releases its shared memory.
                for (uint32_t d = 0; d < RING && d < n_q; ++d) {
                    const uint32_t idx = n_q - 1 - d;
                    mbar_wait_limit(bar(Plan::kBarCode + q * RING + static_cast<int>(idx % RING)), (idx / RING) & 1,
                                    20ll * 1000 * 1000);
                }
            }
        }
    } else {
        // =========================== activation loaders ===========================
        grid_dep_wait();
        const int wl = warp - kTcLoadWarp;  // warps 20 .. 23
        if (p.zero_ptr != nullptr) {  // a later kernel will accumulate into it
            constexpr int ZT = kTcLoadWarps * 32;
            for (long long i = static_cast<long long>(cta) * ZT + wl * 32 + lane; i < p.zero_count;
                 i += static_cast<long long>(gridDim.x) * ZT)
                p.zero_ptr[i] = 0.f;
        }
        if (kTp && p.move_count > 0) {
            constexpr int ZT = kTcLoadWarps * 32;
            for (long long i = static_cast<long long>(cta) * ZT + wl * 32 + lane; i < p.move_count;
                 i += static_cast<long long>(gridDim.x) * ZT) {
                const float v = __ldcg(p.move_src + i);
                p.move_src[i] = 0.f;
                atomicAdd_system(p.move_dst + i, v);  // other ranks may already be adding their products
            }
        }
        // Round r = chunks r * NACC .. r * NACC + NACC - 1 of the CTA's chunk sequence, in round buffer
        // r % NE; loader w owns the buffers b with b % 4 == w (it then meets every phase of their barriers,
        // which is what a parity wait needs).  Slot of (chunk j of the round, k-tile i): (j * C + i) * tile_b.
        // The loader first notes (first k-tile, k-tiles) of the round's chunks in a scratch line of shared
        // memory, then converts all their pieces with several loads in flight per lane.  A piece is 8
        // consecutive k of one row (16 for int8).
        const int M = static_cast<int>(p.M);
        const uint32_t tile_b = tc_tile_bytes<Pol, NMMA>(M);
        const bool bulk = p.x_planes != nullptr;
        const uint8_t *planes = reinterpret_cast<const uint8_t *>(p.x_planes);
        constexpr int LOGR = LOGNACC, RCH = NACC;
        const int NE = tc_rounds<Pol, NMMA>(M);
        const uint32_t round_b = tc_round_bytes<Pol, NMMA>(M);
        volatile int *scratch = reinterpret_cast<volatile int *>(smem_raw + 1024 + wl * 128);  // [RCH][2] ints
        int ci = 0;  // CTA-wide chunk number
        for (int ss = ss_first; ss <= ss_last; ++ss) {
            const int len = seg_len(ss), nchunks = (len + C - 1) / C, kt0 = seg_kt0(ss);
            for (int c = 0; c < nchunks; ++c, ++ci) {
                const int r = ci >> LOGR, j = ci & (RCH - 1);
                const int rb = r % NE;
                if ((rb & (kTcLoadWarps - 1)) != wl) continue;
                const uint32_t rbuf = x_addr + static_cast<uint32_t>(rb) * round_b;
                const int n = len - c * C < C ? len - c * C : C;
                const int kt = kt0 + c * C;  // first k-tile of the chunk
                const bool round_done = j == RCH - 1 || (ss == ss_last && c == nchunks - 1);
                if (j == 0 && r >= NE)  // first chunk of a round: its buffer must have been given back
                    mbar_wait(bar(Plan::kBarXFree + rb), static_cast<uint32_t>(((r / NE) - 1) & 1), flags);
                if (bulk) {
                    // the planes were split once by planes_kernel: a chunk is one contiguous run
                    if (lane == 0) {
                        const uint32_t b = bar(Plan::kBarXReady + rb);
                        const uint32_t bytes = static_cast<uint32_t>(n) * tile_b;
                        asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(b), "r"(bytes) : "memory");
                        bulk_g2s_plain(rbuf + static_cast<uint32_t>(j * C) * tile_b, planes + static_cast<size_t>(kt) * tile_b, bytes, b);
                    }
                    if (round_done) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar(Plan::kBarXReady + rb));
                    }
                    continue;
                }
                if (lane == 0) {
                    scratch[2 * j] = kt;
                    scratch[2 * j + 1] = n;
                }
                if (!round_done) continue;
                __syncwarp();
                // all pieces of the chunks 0 .. j of this round
                const int ppc = kInt ? C * 2 * M : C * 4 * M;  // pieces of a full chunk
                const int ppt = kInt ? 2 * M : 4 * M;          // pieces of a k-tile
                const int total = (j + 1) * ppc;
                constexpr int U = 4;  // pieces in flight per lane
                for (int pbase = 0; pbase < total; pbase += 32 * U) {
                    uint32_t h[U][4];
                    uint32_t dst[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int pid = pbase + u * 32 + lane;
                        dst[u] = 0;
                        if (pid < total) {
                            const int e = pid / ppc, pc = pid - e * ppc, jl = pc / ppt, rem = pc - jl * ppt;
                            const int kte = scratch[2 * e], ne = scratch[2 * e + 1];
                            if (jl < ne) {
                                const uint32_t tdst = rbuf + static_cast<uint32_t>(e * C + jl) * tile_b;
                                if constexpr (kInt) {
                                    const int row = rem >> 1, kh = rem & 1;
                                    const uint4 val = __ldcg(reinterpret_cast<const uint4 *>(
                                        reinterpret_cast<const int8_t *>(p.x) + static_cast<long long>(row) * p.x_ld + 32 * (kte + jl) + 16 * kh));
                                    h[u][0] = val.x; h[u][1] = val.y; h[u][2] = val.z; h[u][3] = val.w;
                                    dst[u] = tdst + kh * (tile_b / 2) + row * 16;
                                } else {
                                    const int row = rem >> 2, kc = rem & 3;
                                    dst[u] = tdst + (kc >> 1) * (tile_b / 2) + row * 16 + (kc & 1) * 8;
                                    load_piece(p.x, p.x_mode, p.x_ld, p.x_gap, row, 32ll * (kte + jl) + 8 * kc, h[u]);
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        if (dst[u] != 0) {
                            if constexpr (kInt) {
                                sts128(dst[u], make_uint4(h[u][0], h[u][1], h[u][2], h[u][3]));
                            } else {
#pragma unroll
                                for (int pl = 0; pl < 4; ++pl) {
                                    const uint2 b8 = next_plane(h[u]);
                                    sts64(dst[u] + pl * (tile_b / 8), b8.x, b8.y);
                                }
                            }
                        }
                    }
                }
                // publish the round
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(Plan::kBarXReady + rb));
            }
        }
        if (bulk && flags[0] && lane == 0) {  // a wait gave up: let the copies in flight land before the CTA exits
            for (int rb = wl; rb < NE; rb += kTcLoadWarps) mbar_wait_limit(bar(Plan::kBarXReady + rb), 0, 2ll * 1000 * 1000);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kTcMmaWarp) tmem_dealloc(tmem, 512);
}

template <class Pol, int NMMA>
inline int launch_tc(const UmmaParams &params, int num_sms, bool pdl, cudaStream_t stream) {
    using Plan = TcPlan<Pol, NMMA>;
    auto kernel = dmm_kernel<Pol, NMMA, false>;
    const bool tp_variant = params.n_peers > 0 || params.move_count > 0;
    if (tp_variant) kernel = dmm_kernel<Pol, NMMA, true>;
    // the shared-memory attribute is set once per kernel variant and device, not on every launch
    static std::atomic<unsigned long long> attr_done[2];
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev >= 64 || !((attr_done[tp_variant ? 1 : 0].load(std::memory_order_acquire) >> dev) & 1ull)) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Plan::kDynBytes));
        if (err != cudaSuccess) return err;
        if (dev < 64) attr_done[tp_variant ? 1 : 0].fetch_or(1ull << dev, std::memory_order_release);
    }
    TcArgs args = {};
    UmmaParams &p = args.p;
    p = params;
    p.dyn_smem_bytes = Plan::kDynBytes;
    const long long KT = p.K / 32, NS = p.N / 16, SST = (NS + 15) / 16;
    const long long T = SST * KT;
    if (T >= (1ll << 31)) return DMM_ERR_SHAPE;
    unsigned grid = static_cast<unsigned>(num_sms);
    if (T < num_sms) grid = static_cast<unsigned>(T);
    p.part.a = static_cast<int>(T / grid);
    p.part.b = static_cast<int>(T % grid);
    if (p.next_codes != nullptr) {
        const long long Tn = ((p.next_N / 16 + 15) / 16) * (p.next_K / 32);
        const long long gn = Tn < num_sms ? Tn : num_sms;
        if (Tn >= (1ll << 31) || gn <= 0) {
            p.next_codes = nullptr;
        } else {
            p.next_grid = static_cast<int>(gn);
            p.next_part.a = static_cast<int>(Tn / gn);
            p.next_part.b = static_cast<int>(Tn % gn);
        }
    }
    const int rc = make_codes_map(&args.map, p.codes, p.N, p.K, Plan::kC);
    if (rc) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kTcThreads);
    cfg.dynamicSmemBytes = Plan::kDynBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args);
}

// fp16 family, 17 to 32 batch rows per launch (128 MMA columns).  The kernel template also compiles
// for the narrower variants and for the int8 policy, but the kernel of dmm_umma.cuh measured faster
// there (28672 x 8192, microseconds, this kernel / that one: batch 1 21.1 / 20.2, batch 16 27.2 / 26.6,
// int8 batch 8 27.6 / 25.2; batch 32 34.2 / 38.7), so only this instantiation is built.
inline int launch_tc_wide(const UmmaParams &p, int num_sms, bool pdl, cudaStream_t stream) {
    return launch_tc<PolF8, 128>(p, num_sms, pdl, stream);
}

}  // namespace dmm
