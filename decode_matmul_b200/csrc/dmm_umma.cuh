// tcgen05 decode-matmul kernel (both families, every batch size) and its small companions.
//
// The decoded weights are the A operand of tcgen05.mma and never touch shared memory: each
// decoder thread owns two output rows, decodes their codes in registers and writes them into
// tensor memory with tcgen05.st; the activations are the B operand, staged in shared memory in
// the canonical no-swizzle K-major layout; accumulators live in TMEM.
//
// Operand policies that share the kernel:
//   PolF8   fp16 family, what the library picks.  Weights as fp6 E2M3 bytes (sign << 5 | |q|,
//           value q/8: exact, and produced by the table XOR alone, 7 instructions per code),
//           the fp16 activations split EXACTLY into four E5M2 planes (the top byte of the half,
//           then of the remainder, ...), kind::f8f6f4, K = 32.  The planes are stacked along
//           the MMA n dimension (N = 16 / 32 / 64 / 128 columns for up to 2 / 8 / 16 / 32 batch
//           rows; up to 2 rows the densely packed planes fit one 8-row core matrix), so
//           one MMA per k-tile does all of them and the epilogue adds the four column groups.
//           Up to 3 batch rows the loader warps split the activations themselves; from 4 rows
//           on planes_kernel splits them once per call and the loaders only issue bulk copies.
//   PolI8   integer family (the reference's operator).  Weights as two's-complement bytes,
//           int8 activations as they are, kind::i8 into int32 accumulators, N = 16 / 32.
//   PolF16  fp16 family, fp16 operands (DMM_PATH_TCGEN05): weights as fp16 integers q (byte ->
//           half by magic number), activations as fp16, kind::f16, K = 16.  A cross-check.
//   PolF8Fast / PolI8Fast: the same over codes in the layout of fast_decode_matmul_cuda.
// Template flags: kChain (several dependent products in one cooperative launch, the CTAs stay
// resident), kTp (tensor-parallel forms: epilogue that adds into every rank's buffer, producer
// and consumer of the slots form) and kSplit (four TMA producer warps, batch 1 and 2).
// Companions in this file: planes_kernel, xrank_barrier_kernel, xrank_allreduce_kernel,
// tp_finalize_kernel.  Batch 17..32 of the fp16 family runs on dmm_kernel (dmm_tc.cuh).
//
// Work decomposition.  A super-tile is 16 strips = 256 output rows = two M=128 MMA tiles:
// tile 0 holds strip rows 0..7 (h = 0) and tile 1 strip rows 8..15 (h = 1) of the 16 strips,
// because one 16-byte piece of the tiled code stream holds the codes of rows g and g+8 and a
// thread decodes both.  A "tile" of work is (super-tile, k-tile): 2 KiB of codes.  Tiles are
// numbered super-tile-major and split evenly and contiguously over the CTAs (stream-K); the
// part of a super-tile a CTA owns is a segment.
//
// Warp roles (25 warps; 28 with kSplit):
//   0..15  decoders, four groups of four warps.  Group q takes the chunks whose CTA-wide number
//          is q mod 4 (C k-tiles of 16 strips each).  Warp wq of a group owns TMEM lanes
//          32wq..32wq+31 = strips 4wq..4wq+3; it reads its strips from the group's code ring,
//          decodes, writes A stage buffers in TMEM and signals the group's MMA issuer.  The
//          decoders also build the look-up table at the start, and groups 0 and 1 run the
//          epilogue of MMA tile 0 and tile 1.
//   16..19 MMA issuers (converged warp, one elected lane issues); issuer s serves the decoder
//          groups q with q % kNAcc == s and owns accumulator s of both MMA tiles (fp8 policy:
//          one issuer per group).  Warp 16 also allocates the tensor memory.
//   20..23 activation loaders (fp8 policy: two teams filling alternate epochs of E5M2 planes;
//          fp16 policy: warps 20 and 21 stage the chunks with cp.async).  They are the only
//          warps that wait for the previous kernel of the stream.
//   24     TMA producer (one thread): streams the code chunks into the groups' rings, one
//          tiled bulk-tensor load per chunk (kSplit: warps 24..27, one per decoder group).
// Every wait is bounded (mbar_wait); nothing spins on another CTA.
#pragma once
#include <cuda.h>

#include <atomic>
#include <functional>
#include <unordered_map>
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
// One lane of the (converged) warp: true in exactly one thread.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n.reg .b32 rx;\n.reg .pred px;\nelect.sync rx|px, 0xffffffff;\nselp.u32 %0, 1, 0, px;\n}\n"
        : "=r"(pred));
    return pred != 0;
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
__device__ __forceinline__ uint32_t tmem_ld1(uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    return r;
}
// wait::ld that also names the loaded registers, so that no use of them can be moved above it
__device__ __forceinline__ void tmem_wait_ld(uint32_t (&r)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
                   "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :
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
// The same with the descriptor as two 32-bit words (only the low word changes from tile to tile).
template <bool kInt = false>
__device__ __forceinline__ void mma_ts_f8_lh(uint32_t d, uint32_t a, uint32_t desc_lo, uint32_t desc_hi, uint32_t idesc,
                                             uint32_t acc) {
    if constexpr (kInt) {
        asm volatile(
            "{\n.reg .pred p;\n.reg .b64 bd;\nsetp.ne.b32 p, %5, 0;\nmov.b64 bd, {%2, %3};\n"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], bd, %4, p;\n}\n" ::"r"(d),
            "r"(a), "r"(desc_lo), "r"(desc_hi), "r"(idesc), "r"(acc)
            : "memory");
        return;
    }
    asm volatile(
        "{\n.reg .pred p;\n.reg .b64 bd;\nsetp.ne.b32 p, %5, 0;\nmov.b64 bd, {%2, %3};\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], bd, %4, p;\n}\n" ::"r"(d),
        "r"(a), "r"(desc_lo), "r"(desc_hi), "r"(idesc), "r"(acc)
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

// The code words of one k-tile for a decoder thread, from a ring slot in the layout of fast_decode_matmul_cuda:
// slot = [8 row blocks of 32][C k-tiles][2 code pairs][32 lanes] uint32, word = two consecutive codes of one
// row.  The thread owns row `lane` of row block wq (MMA tile 0) and of row block wq + 4 (MMA tile 1); the
// words are returned in the form the tile layout delivers them (low half: tile 0's row, high half: tile 1's
// row, one word per code column), so that the decode that follows is the same for both layouts.
__device__ __forceinline__ uint4 fetch_fast_ktile(uint32_t slot_addr, int c_tiles, int wq, int lane, int kt) {
    const uint32_t a = slot_addr + static_cast<uint32_t>(wq * c_tiles + kt) * 256u + static_cast<uint32_t>(lane) * 4u;
    const uint32_t b = a + static_cast<uint32_t>(4 * c_tiles) * 256u;
    const uint32_t a0 = lds32(a), a1 = lds32(a + 128u), b0 = lds32(b), b1 = lds32(b + 128u);
    return make_uint4(prmt(a0, b0, 0x5410u), prmt(a0, b0, 0x7632u), prmt(a1, b1, 0x5410u), prmt(a1, b1, 0x7632u));
}

// ----------------------------------- policies -----------------------------------------
// kG  k-tiles per "group": the unit of decoder -> issuer hand-over (one barrier round trip,
//     one tcgen05.commit).  Every tcgen05 instruction costs its issuing thread ~45-55 cycles
//     whatever its size, so hand-overs and commits are amortised over as many MMAs as fit.
// kNA group buffers per decoder group in TMEM;  kC k-tiles per TMA chunk (multiple of kG).
struct PolF8 {
    static constexpr int kIsF8 = 1;
    static constexpr int kIsInt = 0;
    static constexpr int kFast = 0;    // 1: the codes are in the layout of fast_decode_matmul_cuda (see PolF8Fast)
    static constexpr int kFmt = kFmtFp6;
    static constexpr int kG = 2;
    static constexpr int kNA = 2;
    static constexpr int kC = 4;
    static constexpr int kRing = 3;    // chunks in flight per decoder group
    static constexpr int kACols = 8;   // TMEM columns of one k-tile of one MMA tile (32 k x 1 byte)
    static constexpr uint32_t x_tile_bytes(int) { return 1024; }  // 2 k-halves x (4 planes x 8 rows) x 16 B
    static constexpr int out_cols(int nmma) { return nmma / 4; }    // batch columns per launch: 8 or 16
};
// Integer family (the reference's own operator: int8 activations, int32 result, exact): the
// structure of the fp8 policy -- epoch-resident activations, four accumulator sets -- with the
// weights as two's-complement bytes straight from the table XOR, the int8 activations copied as
// they are (one "plane", the batch rows are the MMA columns) and kind::i8 MMAs into int32.
struct PolI8 {
    static constexpr int kIsF8 = 1;
    static constexpr int kIsInt = 1;
    static constexpr int kFast = 0;
    static constexpr int kFmt = kFmtTwos;
    static constexpr int kG = 2;
    static constexpr int kNA = 2;
    static constexpr int kC = 4;
    static constexpr int kRing = 3;
    static constexpr int kACols = 8;   // 32 k x 1 byte
    static constexpr uint32_t x_tile_bytes(int) { return 1024; }
    static constexpr int out_cols(int nmma) { return nmma; }       // batch columns per launch
};
struct PolF16 {
    static constexpr int kIsF8 = 0;
    static constexpr int kIsInt = 0;
    static constexpr int kFast = 0;
    static constexpr int kFmt = kFmtOffset;
    static constexpr int kG = 1;
    static constexpr int kNA = 2;
    static constexpr int kC = 2;
    static constexpr int kRing = 6;
    static constexpr int kACols = 16;  // 32 k x 2 bytes
    static constexpr uint32_t x_tile_bytes(int nmma) { return static_cast<uint32_t>(nmma) * 64u; }  // 4 k-chunks x rows x 16 B
    static constexpr int out_cols(int nmma) { return nmma; }
};
// The same kernels over codes in the layout of fast_decode_matmul_cuda: their own instantiations, so that the
// tile-layout kernels carry nothing of it (a run-time switch in the decoders' inner loop cost them 9 %).
struct PolF8Fast : PolF8 {
    static constexpr int kFast = 1;
};
struct PolI8Fast : PolI8 {
    static constexpr int kFast = 1;
};

constexpr int kUDecWarps = 16, kUMmaWarp = 16, kUMmaWarps = 4, kULoadWarps = 4, kULoadTeams = 2, kUTmaWarp = 24, kUTmaWarps = 4;
constexpr int kUThreads = (kUDecWarps + kUMmaWarps + kULoadWarps + kUTmaWarps) * 32;
constexpr int kFirstEpoch = 16;  // k-tiles in the first activation epoch of a CTA at batch 1 (fp8 policy)
constexpr int kMaxEpoch = 48;    // and at most this many in the later ones: short epochs keep the
                                 // loaders' latency per epoch below the time the previous one lasts

// k-tiles of the first epoch: one 16-byte piece per thread of a loader team (4 * M pieces per tile)
__host__ __device__ inline int first_epoch_tiles(int E, int M, int ntiles) {
    // (batch 1 with a long tile sequence: 8 measured better than 16, 4 and 2; short sequences: one epoch of 16)
    int e0 = (M == 1 && ntiles >= 64) ? kFirstEpoch / 2 : (kFirstEpoch / M) & ~1;
    if (e0 < 2) e0 = 2;
    return e0 < E ? e0 : E;
}

// Bytes of the E5M2 planes of one k-tile: [k-half][plane][row][16 B].  Up to 8 batch rows the
// rows of a plane are packed densely (M rows); the 64- and 128-column variants pad a plane to 16
// and 32 rows.
template <int NMMA, bool kInt = false>
__host__ __device__ inline uint32_t plane_tile_bytes(int M) {
    if (kInt) return 32u * static_cast<uint32_t>(NMMA);  // int8: [k-half][row < NMMA][16 B], rows padded to the MMA width
    return 128u * static_cast<uint32_t>(NMMA > 64 ? 32 : (NMMA > 32 ? 16 : M));
}

// k-tiles per activation epoch: what fits in one epoch buffer, even, at most kMaxEpoch
__host__ __device__ inline int epoch_tiles(uint32_t epoch_bytes, uint32_t tile_bytes) {
    const int fit = static_cast<int>((epoch_bytes / tile_bytes) & ~1u);
    return fit < kMaxEpoch ? fit : kMaxEpoch;
}
constexpr uint32_t kUBarBytes = 2048;
constexpr uint32_t kUTmemCols = 512;

template <class Pol, int NMMA>
struct UmmaPlan {
    // accumulators per MMA tile = active issuers: one per decoder group while the TMEM holds them
    static constexpr int kNAcc = !Pol::kIsF8 ? 2 : (NMMA <= 32 ? 4 : (NMMA <= 64 ? 2 : 1));
    static constexpr int kNA = Pol::kNA;
    // issuer warps per accumulator: with fewer than four accumulators the two MMA tiles of a
    // group are issued by different warps (each accumulator still has exactly one issuer, so the
    // summation order stays fixed)
    static constexpr int kTileParts = kNAcc <= 2 ? 2 : 1;
    // accumulator sets: with 16 MMA columns two sets fit next to the weight slots, and the segments of a CTA
    // (the parts of different super-tiles in its tile range) alternate between them, so that the epilogue of
    // one segment runs while the MMAs of the next are already being issued
    static constexpr int kSets = (Pol::kIsF8 && !Pol::kIsInt && NMMA == 16) ? 2 : 1;
    static constexpr uint32_t kSetCols = 2 * kNAcc * NMMA;        // one set: both MMA tiles of every accumulator
    static constexpr uint32_t kDCols = kSetCols * kSets;          // TMEM: accumulators first
    static constexpr uint32_t kBufCols = 2 * Pol::kG * Pol::kACols;  // one group buffer: [tile][k-tile][cols]
    static constexpr uint32_t kACols = 4 * kNA * kBufCols;
    static_assert(kDCols + kACols <= kUTmemCols, "TMEM plan exceeds 512 columns");
    static constexpr int kSlots = 4 * kNA;                   // group buffers (= fp16 activation stages)
    static constexpr uint32_t kXStage = Pol::kG * Pol::x_tile_bytes(NMMA);
    // fp8 policy: the activation planes of a whole run of k-tiles ("epoch") stay resident in one
    // of kEpochs buffers, densely packed [tile][k-half][plane][row < M][16 B]
    // (128 columns = 32 batch rows: a k-tile of planes is 4 KiB; an epoch is then one chunk)
    static constexpr int kEpochs = NMMA > 64 ? 3 : 4;
    static constexpr uint32_t kEpochBytes = NMMA > 64 ? 16384 : 14336;
    static constexpr uint32_t kXBytes = Pol::kIsF8 ? kEpochs * kEpochBytes + 256 : kSlots * kXStage;
    static constexpr int kNB = Pol::out_cols(NMMA);               // output columns per launch
    static constexpr uint32_t kPreBytes = kUBarBytes + kXBytes;
    static constexpr uint32_t kSlotBytes = 16 * Pol::kC * 128;    // ring slot: 16 strips x C k-tiles (one TMA box)
    static constexpr uint32_t kRingBytes = 4 * Pol::kRing * kSlotBytes;  // one ring per decoder group
    static constexpr uint32_t kDynBytes = 0x10000u - 0x400u + kLutBytes + kRingBytes;
    static constexpr int kPartial = 2 * kNB * 128;                // output values per segment
    static_assert(kPreBytes <= 0x10000u - 0x400u, "activation stages do not fit below the table");
    static_assert(kDynBytes <= 232448u, "shared memory plan exceeds the per-CTA limit");
    static_assert(Pol::kC % Pol::kG == 0, "a chunk must hold whole groups");
    // barrier indices
    static constexpr int kBarCode = 0;                                   // [4][kRing] TMA completion
    static constexpr int kBarEmpty = kBarCode + 4 * Pol::kRing;          // [4][kRing] the group's 4 warps are done
    static constexpr int kBarFull = kBarEmpty + 4 * Pol::kRing;          // [kSlots] decoder warps (+ fp16 loader)
    static constexpr int kBarFree = kBarFull + kSlots;                   // [kSlots] tcgen05.commit
    static constexpr int kBarXReady = kBarFree + kSlots;                 // [kEpochs] loader warps
    static constexpr int kBarXFree = kBarXReady + kEpochs;               // [kEpochs] both issuers (commit)
    static constexpr int kBarDReady = kBarXFree + kEpochs;
    static constexpr int kBarDFree = kBarDReady + kSets;  // [kSets] each, one per accumulator set
    static constexpr int kBarGridOk = kBarDFree + kSets;  // chains: this CTA's loaders have seen the previous op complete
    static constexpr int kBarCount = kBarGridOk + 1;
    static_assert(kBarCount * 8 + 64 <= kUBarBytes, "barrier block too small");
};

// How the activation loaders read their input (fp8 policy): plain fp16, or fp32 produced by
// the previous layer and converted on the fly, optionally through silu(a) * b of two halves.
constexpr int kXHalf = 0, kXFloat = 1, kXSiluMul = 2;

struct UmmaParams {
    const void *x;       // x_mode 0: fp16 [M, K]; 1: fp32 [M, x_ld]; 2: fp32 [M, x_ld], gate at k, up at x_gap + k
    const void *codes;   // tiled codes
    const void *cb;      // fp16 [256, 8]
    float *out;          // [M, N]
    float *partials;     // workspace [grid][2][kPartial]
    unsigned *tickets;   // workspace, one per super-tile, zero between launches
    long long M, N, K;
    int x_mode;
    long long x_ld, x_gap;  // row stride of x in elements; offset of the second operand (mode 2)
    float scale;         // includes the unit of the accumulators (1/4 for q, 2 for q/8)
    int accumulate;
    int atomic_reduce;   // partial super-tiles are added to `out` with red.global.add (out must hold the
                         // value to add to): no workspace round trip, summation order not fixed
    int sign_convention;
    const void *x_planes;  // fp8 policy, optional: the E5M2 planes of x already split by planes_kernel, in the
                           // layout of the epoch buffers ([k-tile][k-half][plane][row][16 B]); the
                           // kernel then copies them with bulk copies and its loaders do no arithmetic
    // Tensor-parallel epilogue (optional): with n_peers > 0 the atomic adds go to the same buffer on
    // every rank (peer_out[r], this rank's own included) instead of `out`, over NVLink peer memory,
    // so that the sum over ranks needs no separate all-reduce; see dmm_f16_fused_tp.
    float *peer_out[8];
    int n_peers;
    // Tensor-parallel "slots" form (tp_mode 2 = producer, 3 = consumer; see dmm_f16_tp_produce / _consume):
    // peer_out[r] is then the base of rank r's slot array [2 parities][world][tp_count] and tp_flags[r] its
    // flag words; words 16 and 17 of this rank's own flag array are its epoch counter and arrival ticket.
    int tp_mode, tp_rank, tp_world;
    unsigned *tp_flags[8];
    long long tp_count;    // floats per slot = M * N of the row-parallel products
    long long tp_wait;     // clock cycles after which the consumer's flag wait gives up
    float *h_out;          // consumer: where the summed residual stream is written ([M, x_ld])
    float *move_src;     // optional: move_dst[i] += move_src[i], then move_src[i] = 0 (this rank's copy of the
    float *move_dst;     // residual stream changing buffers), done by the loaders like the clearing below
    long long move_count;
    float *zero_ptr;     // optional: buffer this kernel clears on its way (see dmm_f16_fused)
    long long zero_count;
    Part32 part;         // tiles per CTA: part.a = T / grid, part.b = T % grid
    unsigned dyn_smem_bytes;
    // Optional hint: the code matrix of the NEXT product of the stream (dmm_hint_next_weights).  When this
    // kernel's TMA producers have issued their last load they fetch, into L2 only, the first ring fill that
    // CTA `blockIdx.x` of that next launch will ask for, so that its first codes -- the longest wait of a
    // launch's prologue -- come from L2 instead of DRAM.
    int fast_layout;     // codes are in the layout of fast_decode_matmul_cuda (fp8/int8 policies stream it natively)
    const void *next_codes;
    long long next_N, next_K;
    Part32 next_part;
    int next_grid;
};

// Accumulator element of the epilogue: fp32, or int32 for the integer family.
template <bool kInt> struct AccType { using type = float; };
template <> struct AccType<true> { using type = int; };
template <class Acc> __device__ __forceinline__ Acc acc_from_bits(uint32_t r);
template <> __device__ __forceinline__ float acc_from_bits<float>(uint32_t r) { return __uint_as_float(r); }
template <> __device__ __forceinline__ int acc_from_bits<int>(uint32_t r) { return static_cast<int>(r); }
__device__ __forceinline__ float acc_scaled(float scale, float v) { return scale * v; }
__device__ __forceinline__ int acc_scaled(float, int v) { return v; }

// Several dependent products in one launch ("chain"): op k+1 reads what op k wrote.  The CTAs
// stay resident; between two ops only the activation loaders wait (for every CTA to have
// finished op k, counted in `sync`), while the decoders already work on the weights of op k+1.
constexpr int kMaxOps = 8;
template <int kOps>
struct UmmaChainT {
    UmmaParams op[kOps];
    CUtensorMap map[kOps];
    int n_ops;
    unsigned *sync;  // [n_ops] arrival counters in global memory, zero between launches (chains only)
};

// Residual stream plus the partial products that every rank of a tensor-parallel group has pushed into
// this rank's slots (consumer side of the slots form): eight consecutive values of one row, summed in
// rank order; the sum is also written to h_out, and returned rounded to fp16.
__device__ __forceinline__ void load_piece_sum(const float *h_in, float *h_out, const float *slots, int world,
                                               long long slot_stride, long long x_ld, int row, long long k0, uint32_t (&h)[4]) {
    const long long off = row * x_ld + k0;
    float4 a0 = __ldcg(reinterpret_cast<const float4 *>(h_in + off));
    float4 a1 = __ldcg(reinterpret_cast<const float4 *>(h_in + off + 4));
    float4 v0[8], v1[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
        v0[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        v1[r] = v0[r];
        if (r < world) {
            v0[r] = __ldcg(reinterpret_cast<const float4 *>(slots + r * slot_stride + off));
            v1[r] = __ldcg(reinterpret_cast<const float4 *>(slots + r * slot_stride + off + 4));
        }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {  // rank order: every rank computes the same bits
        a0.x += v0[r].x; a0.y += v0[r].y; a0.z += v0[r].z; a0.w += v0[r].w;
        a1.x += v1[r].x; a1.y += v1[r].y; a1.z += v1[r].z; a1.w += v1[r].w;
    }
    *reinterpret_cast<float4 *>(h_out + off) = a0;
    *reinterpret_cast<float4 *>(h_out + off + 4) = a1;
    const float f[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __half2 hh = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
        h[j] = *reinterpret_cast<const uint32_t *>(&hh);
    }
}

// Eight consecutive activations of one row as four packed half2 words, from any input kind.
__device__ __forceinline__ void load_piece(const void *xp, int x_mode, long long x_ld, long long x_gap, int row,
                                           long long k0, uint32_t (&h)[4]) {
    if (x_mode == kXHalf) {
        // (ld.cg: inside a chain the same buffer is rewritten between ops, L1 could hold a stale line)
        const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(xp) + row * x_ld + k0));
        h[0] = v.x; h[1] = v.y; h[2] = v.z; h[3] = v.w;
        return;
    }
    const float *xf = reinterpret_cast<const float *>(xp) + row * x_ld + k0;
    const float4 a0 = __ldcg(reinterpret_cast<const float4 *>(xf));
    const float4 a1 = __ldcg(reinterpret_cast<const float4 *>(xf + 4));
    float f[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    if (x_mode == kXSiluMul) {
        const float4 b0 = __ldcg(reinterpret_cast<const float4 *>(xf + x_gap));
        const float4 b1 = __ldcg(reinterpret_cast<const float4 *>(xf + x_gap + 4));
        const float g[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = __fdividef(f[j], 1.0f + __expf(-f[j])) * g[j];
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __half2 hh = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
        h[j] = *reinterpret_cast<const uint32_t *>(&hh);
    }
}

// Plane `pl` of a piece = the top byte of each half (an E5M2 number: truncation of the half);
// returns its eight bytes and leaves the exact remainder in h for the next plane.
__device__ __forceinline__ uint2 next_plane(uint32_t (&h)[4]) {
    const uint2 bytes = make_uint2(prmt(h[0], h[1], 0x7531u), prmt(h[2], h[3], 0x7531u));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t top = h[j] & 0xFF00FF00u;
        __half2 rr = __hsub2(*reinterpret_cast<__half2 *>(&h[j]), *reinterpret_cast<const __half2 *>(&top));
        h[j] = *reinterpret_cast<uint32_t *>(&rr);
    }
    return bytes;
}

// Barrier between the ranks of a tensor-parallel group, one process per GPU: thread t tells rank t
// that this rank has arrived (a release store of the barrier's number into slot `rank` of rank t's
// flag array, through peer memory) and waits, bounded, until rank t has told this rank the same.
// The number comes from a counter in this GPU's memory that every execution increments, so a
// captured launch can be replayed.  The ranks are different GPUs, hence run concurrently.
struct XrankBarrierParams {
    unsigned *flags[8];  // flags[t]: rank t's array of `world` words (peer pointers; [rank] is local)
    unsigned *counter;   // this rank's barrier counter (local)
    int rank, world;
    long long wait_limit;  // clock cycles after which the wait gives up (DMM_STATUS_WAIT_TIMEOUT)
};
__global__ void __launch_bounds__(32) xrank_barrier_kernel(const XrankBarrierParams bp) {
    // Launched with programmatic stream serialization: the kernel after it may start at once (its
    // weight decode does not depend on other ranks; its activation loaders wait for this kernel to
    // finish), and this kernel itself may have started before the one before it has finished.
    grid_dep_launch();
    grid_dep_wait();
    const int t = threadIdx.x;
    unsigned e = 0;
    if (t == 0) e = atomicAdd(bp.counter, 1u) + 1u;
    e = __shfl_sync(0xffffffffu, e, 0);
    __threadfence_system();  // everything this GPU wrote before (peer atomics of the kernel before) first
    if (t < bp.world) {
        unsigned *dst = bp.flags[t] + bp.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(e) : "memory");
        const unsigned *mine = bp.flags[bp.rank] + t;
        const long long t0 = clock64();
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (static_cast<int>(v - e) >= 0) break;
            if (clock64() - t0 > bp.wait_limit) {
                raise_status(DMM_STATUS_WAIT_TIMEOUT);
                break;
            }
            __nanosleep(100);
        }
    }
    __threadfence_system();
}

// One-shot all-reduce-and-add for the tensor-parallel step: every rank has accumulated its partial
// [count] fp32 product into its own `src` buffer (peer_src[r] = that buffer on rank r, mapped
// through peer memory); this kernel waits until all ranks have got that far (the barrier of
// xrank_barrier_kernel, signalled by block 0, awaited by every block on this rank's own flag words),
// then each rank PULLS the partials of all ranks with coalesced 16-byte loads over NVLink, adds them
// in rank order (so every rank computes the same bits) and adds the sum to its local `dst`.  It also
// clears `zero_local`, the partial buffer of the layer before: all ranks have finished reading it
// once they have signalled this barrier.  The barrier number is the device counter + 1, read by every
// block before the last block to finish increments it.
struct XrankAllreduceParams {
    const float *peer_src[8];
    unsigned *flags[8];
    unsigned *counter;   // this rank's count of finished all-reduces (local)
    unsigned *ticket;    // this rank's count of finished blocks of the running kernel (local, zero between kernels)
    float *dst;          // local
    float *zero_local;   // local, may be null
    long long count;     // floats, multiple of 4
    int rank, world;
    long long wait_limit;  // clock cycles after which the wait gives up (DMM_STATUS_WAIT_TIMEOUT)
};
__global__ void __launch_bounds__(256) xrank_allreduce_kernel(const XrankAllreduceParams ap) {
    grid_dep_launch();
    grid_dep_wait();
    __shared__ int failed;
    const int t = threadIdx.x;
    if (t == 0) failed = 0;
    const unsigned e = *reinterpret_cast<volatile const unsigned *>(ap.counter) + 1u;
    __syncthreads();
    if (blockIdx.x == 0 && t < ap.world) {
        __threadfence_system();
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ap.flags[t] + ap.rank), "r"(e) : "memory");
    }
    if (t < ap.world) {
        const unsigned *mine = ap.flags[ap.rank] + t;
        const long long t0 = clock64();
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if (static_cast<int>(v - e) >= 0) break;
            if (clock64() - t0 > ap.wait_limit) {
                raise_status(DMM_STATUS_WAIT_TIMEOUT);
                failed = 1;
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    if (!failed) {
        const long long n4 = ap.count / 4;
        for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + t; i < n4;
             i += static_cast<long long>(gridDim.x) * blockDim.x) {
            // all ranks' loads go out before the first one is used: one NVLink round trip, not `world`
            float4 v[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                v[r] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (r < ap.world)
                    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
                                 : "=f"(v[r].x), "=f"(v[r].y), "=f"(v[r].z), "=f"(v[r].w)
                                 : "l"(reinterpret_cast<const float4 *>(ap.peer_src[r]) + i));
            }
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int r = 0; r < 8; ++r) {  // rank order: every rank computes the same bits
                acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w;
            }
            float4 *d = reinterpret_cast<float4 *>(ap.dst) + i;
            float4 o = *d;
            o.x += acc.x; o.y += acc.y; o.z += acc.z; o.w += acc.w;
            *d = o;
            if (ap.zero_local != nullptr) reinterpret_cast<float4 *>(ap.zero_local)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    // the last block to finish moves the counter on (every block has read it by then)
    __threadfence();
    __syncthreads();
    if (t == 0) {
        const unsigned done = atomicAdd(ap.ticket, 1u);
        if (done == gridDim.x - 1) {
            *ap.ticket = 0;
            __threadfence();
            atomicAdd(ap.counter, 1u);
        }
    }
}

// End of a tensor-parallel step in the slots form: h_out = h_in + the partial products of the last epoch
// from every rank's slot (what a consumer's loaders do on the fly, as a kernel of its own).
struct TpFinalizeParams {
    const float *h_in;
    float *h_out;
    const float *slots;      // this rank's slot array [2][world][count]
    const unsigned *flags;   // this rank's flag words; word 16 = epoch counter
    long long count;
    int world;
    long long wait_limit;
};
__global__ void __launch_bounds__(256) tp_finalize_kernel(const TpFinalizeParams fp) {
    grid_dep_launch();
    grid_dep_wait();
    const int t = threadIdx.x;
    const unsigned e = *reinterpret_cast<volatile const unsigned *>(fp.flags + 16);
    if (t < fp.world) {
        const long long t0 = clock64();
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(fp.flags + t) : "memory");
            if (static_cast<int>(v - e) >= 0) break;
            if (clock64() - t0 > fp.wait_limit) {
                raise_status(DMM_STATUS_WAIT_TIMEOUT);
                break;
            }
            __nanosleep(40);
        }
    }
    __syncthreads();
    const float *sl = fp.slots + static_cast<long long>(e & 1u) * fp.world * fp.count;
    const long long n4 = fp.count / 4;
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + t; i < n4; i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float4 a = __ldcg(reinterpret_cast<const float4 *>(fp.h_in) + i);
        float4 v[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            v[r] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (r < fp.world) v[r] = __ldcg(reinterpret_cast<const float4 *>(sl + r * fp.count) + i);
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            a.x += v[r].x; a.y += v[r].y; a.z += v[r].z; a.w += v[r].w;
        }
        reinterpret_cast<float4 *>(fp.h_out)[i] = a;
    }
}

// Splits the activations of one call into E5M2 planes ONCE, in the layout the tcgen05 kernel's
// epoch buffers use: [k-tile][k-half][plane][row < rows_padded][16 B].  With more than a few
// batch rows the per-CTA split inside umma_kernel (every CTA repeats it for its k range) costs
// more than the decode itself; this kernel does it once and umma_kernel then only copies.
// One thread per piece (8 k of one row); thread order (k-tile, k-half, row, half) so that the
// stores of a warp are contiguous per plane.
__global__ void __launch_bounds__(128) planes_kernel(const void *x, int x_mode, long long x_ld, long long x_gap, int M,
                                                     long long K, int rows_padded, uint8_t *planes) {
    grid_dep_wait();  // x is the previous kernel's output; the buffer may still be read by the kernel before it
    grid_dep_launch();
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const int per_half = 2 * M;  // pieces per (k-tile, k-half)
    const long long kh_idx = idx / per_half;
    if (kh_idx >= K / 16) return;
    const int rem = static_cast<int>(idx - kh_idx * per_half), row = rem >> 1, half = rem & 1;
    uint32_t h[4];
    load_piece(x, x_mode, x_ld, x_gap, row, kh_idx * 16 + half * 8, h);
    const uint32_t tile_b = 128u * static_cast<uint32_t>(rows_padded);
    uint8_t *dst = planes + kh_idx * (tile_b / 2) + row * 16 + half * 8;
#pragma unroll
    for (int pl = 0; pl < 4; ++pl) *reinterpret_cast<uint2 *>(dst + pl * (tile_b / 8)) = next_plane(h);
}

// `codes_map` is a 2-D tensor map of the tiled code matrix: inner dimension = one strip
// (K/32 k-tiles x 32 uint32), outer dimension = strips; box = kC k-tiles x 16 strips.
// kChain == false is the plain single-product kernel: the op loops below run once with every
// per-op value a compile-time-known kernel parameter.
// kTp == true adds the tensor-parallel pieces (adds into every rank's buffer, residual move).
// kSplit == true is the instantiation with four TMA producer warps (28 warps; the register budget per
// thread is smaller, which only the 32-column fp16-family kernel tolerates without a slow-down).
template <class Pol, int NMMA, bool kChain, bool kTp = false, bool kSplit = false>
__global__ void __launch_bounds__(kSplit ? kUThreads : kUThreads - (kUTmaWarps - 1) * 32, 1) umma_kernel(const __grid_constant__ UmmaChainT<kChain ? kMaxOps : 1> ch) {
    using Plan = UmmaPlan<Pol, NMMA>;
    constexpr int C = Pol::kC, G = Pol::kG, NA = Plan::kNA, RING = Pol::kRing, NACC = Plan::kNAcc, NB = Plan::kNB;
    constexpr int TP = Plan::kTileParts;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t lut_addr = (base + Plan::kPreBytes + 0xFFFFu) & ~0xFFFFu;
    const uint32_t ring_addr = lut_addr + kLutBytes;
    const uint32_t x_addr = base + kUBarBytes;
    volatile int *flags = reinterpret_cast<volatile int *>(smem_raw + Plan::kBarCount * 8);  // [0]=failed [1]=last
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_raw + Plan::kBarCount * 8 + 16);
    auto bar = [&](int i) -> uint32_t { return base + 8u * static_cast<uint32_t>(i); };

    // the warp index through a shuffle: the compiler then knows it is the same in every lane and
    // keeps what derives from it (roles, descriptors, TMEM addresses) in uniform registers
    const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
    const UmmaParams &p0 = ch.op[0];  // codebook, sign convention, batch and input kind are common to all ops
    const int n_ops = kChain ? ch.n_ops : 1;
    // the codebook is static data: fetch it first (fp16 table; the integer family's int64 table is read in lut_fill)
    const uint4 cb_pre = Pol::kIsInt ? make_uint4(0, 0, 0, 0) : lut_prefetch(p0.cb, tid);

    if (ring_addr + Plan::kRingBytes > base + p0.dyn_smem_bytes) {  // uniform over the grid
        if (tid == 0) raise_status(DMM_STATUS_BAD_SMEM);
        return;
    }

    const int cta = blockIdx.x;
    // Per-op geometry, set by every role at the top of its op loop: this CTA's tiles [i0, i1) of
    // the op's (super-tile, k-tile) sequence and the segments (parts of a super-tile) they span.
#define DMM_OP_GEOMETRY(P)                                                                          \
    const int KT = static_cast<int>((P).K / 32);                                                   \
    const int i0 = part32_begin((P).part, cta), i1 = part32_begin((P).part, cta + 1);              \
    const int ss_first = i0 / KT, ss_last = i1 > i0 ? (i1 - 1) / KT : ss_first - 1;                \
    auto seg_kt0 = [&](int ss) -> int {                                                            \
        const int a = ss * KT;                                                                     \
        return i0 > a ? i0 - a : 0;                                                                \
    };                                                                                             \
    auto seg_len = [&](int ss) -> int {                                                            \
        const int a = ss * KT;                                                                     \
        const int lo = i0 > a ? i0 : a, hi = i1 < a + KT ? i1 : a + KT;                            \
        return hi - lo;                                                                            \
    };                                                                                             \
    auto seg_chunks = [&](int ss) -> int { return (seg_len(ss) + C - 1) / C; };                    \
    (void)seg_kt0; (void)seg_chunks; (void)ss_last
    // Chunks are numbered through all segments and ops of the CTA (cbase = chunks before);
    // chunk number mod 4 is the decoder group and mod kNAcc the issuer, so consecutive chunks
    // always go to different groups, also across a segment or op boundary.

    // ---- set-up ----
    // The decoder warps build the look-up table straight away; the other warps initialise the
    // barriers, allocate TMEM and zero the fp16 activation stages meanwhile and then go on
    // (the code stream starts flowing while the table is still being built).  The decoders
    // join through barrier 4, on which the others only arrive.
    // 25 warps (one TMA producer) or 28 (four, one per decoder group: batch 1 and 2 of the fp16 family)
    constexpr int n_threads = kSplit ? kUThreads : kUThreads - (kUTmaWarps - 1) * 32, n_other = n_threads - kUDecWarps * 32;
    bool bad_cb = false;
    if (warp < kUDecWarps) {
        bad_cb = lut_fill(lut_addr, p0.cb, Pol::kIsInt ? 0 : 1, p0.sign_convention, Pol::kFmt, tid, kUDecWarps * 32,
                          Pol::kIsF8 != 0 && !Pol::kIsInt, Pol::kIsInt ? nullptr : &cb_pre);
        named_barrier(4, n_threads);
    } else {
        const int ot = tid - kUDecWarps * 32;  // 0 .. n_other-1
        const int bt = ot - kUMmaWarps * 32;   // loader and TMA warps initialise the barriers
        if (bt >= 0 && bt < Plan::kBarCount) {
            uint32_t count = 1;                                                // TMA, tcgen05.commit
            if (bt >= Plan::kBarEmpty && bt < Plan::kBarFull) count = 4;
            if (bt >= Plan::kBarFull && bt < Plan::kBarFree) count = Pol::kIsF8 ? 4 : 5;  // decoder warps (+ loader)
            if (bt >= Plan::kBarXReady && bt < Plan::kBarXFree) count = p0.x_planes != nullptr ? 1 : kULoadWarps / kULoadTeams;
            if (bt >= Plan::kBarFree && bt < Plan::kBarXReady) count = TP;  // tcgen05.commit of every issuer of the slot
            if (bt >= Plan::kBarXFree && bt < Plan::kBarDReady) count = NACC * TP;
            if (bt >= Plan::kBarDReady && bt < Plan::kBarDFree) count = NACC * TP;
            if (bt >= Plan::kBarDFree && bt < Plan::kBarGridOk) count = 8;
            if (bt == Plan::kBarGridOk) count = kULoadWarps;
            mbar_init(bar(bt), count);
            if (bt == 0) {
                flags[0] = 0;
                flags[1] = 0;
                flags[2] = 2;
                if constexpr (kTp) {
                    // Slots form: word 18 of a rank's flag array is the epoch in production.  CTA 0 of a producer
                    // sets it before any of its threads lets dependent kernels start; a consumer reads it before
                    // it lets the next producer start, and so never needs to wait for the producer kernel as a
                    // whole -- the producer's flags tell it when the data it reads is complete.
                    if (p0.tp_mode == 2 && cta == 0) {
                        unsigned *w = p0.tp_flags[p0.tp_rank];
                        *reinterpret_cast<volatile unsigned *>(w + 18) = *reinterpret_cast<volatile const unsigned *>(w + 16) + 1u;
                        __threadfence();
                    }
                    if (p0.tp_mode == 3) flags[3] = static_cast<int>(*reinterpret_cast<volatile const unsigned *>(p0.tp_flags[p0.tp_rank] + 18));
                }
            }
            fence_mbar_init();
        }
        if (warp == kUMmaWarp) tmem_alloc(smem_u32(const_cast<uint32_t *>(tmem_slot)), kUTmemCols);
        if constexpr (!Pol::kIsF8) {  // fp16 stages: rows past the batch must read as zero
            for (uint32_t o = ot * 16u; o < Plan::kXBytes; o += n_other * 16u) sts128(x_addr + o, make_uint4(0, 0, 0, 0));
        }
        fence_async_smem();
        tc_fence_before();
        named_barrier(3, n_other);
        named_barrier_arrive(4, n_threads);
    }
    tc_fence_after();
    const uint32_t tmem = __shfl_sync(0xffffffffu, *tmem_slot, 0);
    // (a consumer of the slots form lets the next kernel start only once its loaders have seen the producer's
    // flags: the kernels after it then find that producer's epoch counter moved on)
    if (!(kTp && p0.tp_mode == 3)) grid_dep_launch();

    if (warp < kUDecWarps) {
        // =============================== decoders ===============================
        // Nothing here reads what an earlier kernel of the stream wrote (codes and codebook are
        // static), so the decoders never wait for it: they decode ahead into TMEM while the
        // previous kernel drains; the activation loaders are the ones that wait.
        const int q = warp >> 2, wq = warp & 3;
        const uint32_t gring = ring_addr + static_cast<uint32_t>(q) * (RING * Plan::kSlotBytes);  // ring of group q
        if (bad_cb) raise_status(DMM_STATUS_BAD_CODEBOOK);
        LutLane ll = lut_lane(lut_addr, lane, Pol::kIsF8 != 0 && !Pol::kIsInt);
        ll.two = static_cast<uint32_t>(flags[2]);

        const uint32_t tlane = tmem + (static_cast<uint32_t>(wq * 32) << 16);
        // Tensor-parallel producer: this launch is epoch e = counter + 1 and accumulates into this rank's own
        // slot of parity e & 1.  The counter is read at the first epilogue, i.e. after this kernel's loaders
        // have seen the kernel before it finish (so the producer before this one has moved it on), and stays
        // put until the last CTA of this launch has seen every other CTA finish.
        [[maybe_unused]] unsigned tp_epoch = 0;
        [[maybe_unused]] float *tp_slot_mine = nullptr;
        // The four groups share the shared-memory look-up pipe and are otherwise independent:
        // start them a fraction of a group apart so that one group's hand-over and waiting
        // falls into the others' look-up bursts instead of all groups idling together.
        if (q != 0) __nanosleep(static_cast<unsigned>(q) * 128u);
        uint32_t sA = 0;  // groups this decoder group has produced
        int segidx = 0, ebase = 0;  // segments and chunks of this CTA so far (all ops)
        int cidx = 0;  // chunks this group has consumed
        for (int op = 0; op < n_ops; ++op) {
        const UmmaParams &p = ch.op[op];
        DMM_OP_GEOMETRY(p);
        for (int ss = ss_first; ss <= ss_last; ebase += seg_chunks(ss), ++ss, ++segidx) {
            const int len = seg_len(ss);
            const int nchunks_ss = (len + C - 1) / C;
            for (int c = (q - ebase) & 3; c < nchunks_ss; c += 4) {
                const int n = len - c * C < C ? len - c * C : C;  // k-tiles in this chunk
                const int slot = cidx % RING;
                mbar_wait(bar(Plan::kBarCode + q * RING + slot), static_cast<uint32_t>((cidx / RING) & 1), flags);
                // slot layout [16 strips][C k-tiles][128 B]; this lane: strip 4*wq + lane/8, piece lane%8
                const uint32_t src = gring + slot * Plan::kSlotBytes + (wq * 4 + (lane >> 3)) * (C * 128) + (lane & 7) * 16;
                const uint32_t fsrc = gring + slot * Plan::kSlotBytes;  // (fast layout: see fetch_fast_ktile)
                constexpr bool fast = Pol::kFast != 0;
#pragma unroll 1
                for (int g0 = 0; g0 < n; g0 += G) {
                    const int buf = static_cast<int>(sA % NA);
                    const int sl = q * NA + buf;
                    if (sA >= NA) mbar_wait(bar(Plan::kBarFree + sl), ((sA / NA) - 1) & 1, flags);
                    tc_fence_after();
                    const uint32_t acol = tlane + Plan::kDCols + static_cast<uint32_t>(sl) * Plan::kBufCols;
                    if constexpr (Pol::kIsF8) {
                        // group buffer columns: [tile][k-tile][8]; two k-tiles -> one x16 store per tile
                        uint32_t r0[8 * G], r1[8 * G];
#pragma unroll
                        for (int i = 0; i < G; ++i) {
                            uint4 cw = make_uint4(0, 0, 0, 0);
                            if (g0 + i < n) cw = fast ? fetch_fast_ktile(fsrc, C, wq, lane, g0 + i) : lds128(src + (g0 + i) * 128);
                            const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
                            for (int t = 0; t < 4; ++t) {
                                uint2 d0, d1;
                                if constexpr (Pol::kIsInt) {
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
                        static_assert(G == 2 || !Pol::kIsF8, "fp8 policy stores two k-tiles at once");
                        tmem_st16(acol, reinterpret_cast<const uint32_t(&)[16]>(r0));
                        tmem_st16(acol + G * Pol::kACols, reinterpret_cast<const uint32_t(&)[16]>(r1));
                    } else {
                        const uint4 cw = lds128(src + g0 * 128);
                        const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
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
                        tmem_st16(acol + G * Pol::kACols, r1);
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(Plan::kBarFull + sl));
                    ++sA;
                }
                __syncwarp();  // every lane has read the slot: hand it back to the TMA warp
                if (lane == 0) mbar_arrive(bar(Plan::kBarEmpty + q * RING + slot));
                ++cidx;
            }

            if (q < 2) {
                // ---------------- epilogue of MMA tile q of this segment ----------------
                const int nchunks = nchunks_ss;
                // accumulator a was written in this segment iff one of its chunks has parity a
                uint32_t used = 0;
                for (int cc = 0; cc < nchunks && cc < NACC; ++cc) used |= 1u << ((ebase + cc) % NACC);
                const int aset = segidx % Plan::kSets;  // accumulator set of this segment
                const uint32_t aset_col = static_cast<uint32_t>(aset) * Plan::kSetCols;
                mbar_wait(bar(Plan::kBarDReady + aset), static_cast<uint32_t>((segidx / Plan::kSets) & 1), flags);
                tc_fence_after();
                // the accumulators are fp32, or int32 for the integer family (exact, no scale)
                using Acc = typename AccType<Pol::kIsInt != 0>::type;
                Acc v[NB];
#pragma unroll
                for (int b = 0; b < NB; ++b) v[b] = Acc(0);
                Acc *out_acc = reinterpret_cast<Acc *>(p.out);
                if (kTp && p.tp_mode == 2) {
                    tp_epoch = *reinterpret_cast<volatile const unsigned *>(p.tp_flags[p.tp_rank] + 16) + 1u;
                    tp_slot_mine = p.peer_out[p.tp_rank] + (static_cast<long long>(tp_epoch & 1u) * p.tp_world + p.tp_rank) * p.tp_count;
                    out_acc = reinterpret_cast<Acc *>(tp_slot_mine);
                }
                Acc *const partials_acc = reinterpret_cast<Acc *>(p.partials);
                if (Pol::kIsF8 && !Pol::kIsInt && p.M == 1) {
                    // batch 1: only column 8 * plane of every accumulator carries data (column `plane` in the
                    // 16-column build, whose single core matrix holds all four planes); fetch those
                    // sixteen words with one wait instead of whole accumulators one after the other
                    uint32_t r[16];
#pragma unroll
                    for (int a = 0; a < 4; ++a) {
#pragma unroll
                        for (int pl = 0; pl < 4; ++pl) {
                            r[a * 4 + pl] = 0u;
                            if (a < NACC && ((used >> a) & 1u))
                                r[a * 4 + pl] = tmem_ld1(tlane + aset_col + static_cast<uint32_t>((q * NACC + a) * NMMA + (NMMA == 16 ? 1 : 8) * pl));
                        }
                    }
                    tmem_wait_ld(r);
#pragma unroll
                    for (int e = 0; e < 16; ++e) v[0] += acc_from_bits<Acc>(r[e]);
                } else if (Pol::kIsF8 && !Pol::kIsInt && NMMA == 16) {
                    // 16-column build at batch 2: the planes are packed densely, column 2 * plane + row
#pragma unroll
                    for (int a = 0; a < NACC; ++a) {
                        if ((used >> a) & 1u) {
                            uint32_t r[16];
                            tmem_ld16(tlane + aset_col + static_cast<uint32_t>((q * NACC + a) * NMMA), r);
                            tmem_wait_ld(r);
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e & 1] += acc_from_bits<Acc>(r[e]);
                        }
                    }
                } else {
#pragma unroll
                    for (int a = 0; a < NACC; ++a) {
                        if ((used >> a) & 1u) {
#pragma unroll
                            for (int b0 = 0; b0 < NMMA; b0 += 16) {
                                uint32_t r[16];
                                tmem_ld16(tlane + aset_col + static_cast<uint32_t>((q * NACC + a) * NMMA + b0), r);
                                tmem_wait_ld(r);
                                // PolF8: column 8*plane + b; PolF16: column b
#pragma unroll
                                for (int e = 0; e < 16; ++e) v[(b0 + e) % NB] += acc_from_bits<Acc>(r[e]);
                            }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(Plan::kBarDFree + aset));

                const int ss_a = ss * KT;
                const bool full = len == KT;
                const int my_slot = seg_kt0(ss) > 0 ? 0 : 1;
                const int trow = wq * 32 + lane;  // TMEM lane = row of the MMA tile
                const long long n = Pol::kFast
                                        ? static_cast<long long>(ss) * 256 + 32 * (4 * q + wq) + lane
                                        : (static_cast<long long>(ss) * 16 + wq * 4 + (lane >> 3)) * 16 + 8 * q + (lane & 7);
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
        if (kTp && p.tp_mode == 2 && q < 2) {
            // Tensor-parallel producer, after this CTA's last atomic adds: the last CTA of the grid to get
            // here copies this rank's finished partial product into its slot on every other rank (plain
            // vector stores over NVLink: one value per element and peer) and then raises this rank's flag
            // on every rank to the epoch number.  One NVLink traversal, no barrier, no further kernel.
            __threadfence();
            named_barrier(2, 256);
            const int et = q * 128 + wq * 32 + lane;  // 0 .. 255
            if (et == 0) {
                unsigned *ticket = p.tp_flags[p.tp_rank] + 17;
                const unsigned old = atomicAdd(ticket, 1u);
                const int last = old == gridDim.x - 1;
                if (last) *ticket = 0;
                flags[1] = last;
            }
            named_barrier(2, 256);
            if (flags[1] != 0) {
                __threadfence();
                const long long n4 = p.tp_count / 4;
                const long long slot_off = (static_cast<long long>(tp_epoch & 1u) * p.tp_world + p.tp_rank) * p.tp_count;
                // (eight loads in flight per thread before the first store: the loop is one L2 round trip per
                // 32 KB instead of one per 4 KB)
                for (long long i0 = et; i0 < n4; i0 += 256 * 8) {
                    float4 v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (i0 + u * 256 < n4) v[u] = __ldcg(reinterpret_cast<const float4 *>(tp_slot_mine) + i0 + u * 256);
                    for (int r = 0; r < p.tp_world; ++r) {
                        if (r == p.tp_rank) continue;
                        float4 *dst = reinterpret_cast<float4 *>(p.peer_out[r] + slot_off);
#pragma unroll
                        for (int u = 0; u < 8; ++u)
                            if (i0 + u * 256 < n4) dst[i0 + u * 256] = v[u];
                    }
                }
                if (et == 0) {
                    *reinterpret_cast<volatile unsigned *>(p.tp_flags[p.tp_rank] + 16) = tp_epoch;  // the epoch counter moves on
                }
                // one release per flag covers the stores of all 256 threads (the barrier orders them before it)
                named_barrier(2, 256);
                if (et < p.tp_world)
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.tp_flags[et] + p.tp_rank), "r"(tp_epoch) : "memory");
            }
            named_barrier(2, 256);
        }
        if (n_ops > 1 && q < 2) {
            // Chain: tell the other CTAs that this one has finished op `op` (all its atomic adds
            // are out), once its own loaders have seen op - 1 complete -- the last CTA to arrive
            // here then knows that nobody polls the counter of op - 1 any more and clears it.
            __threadfence();
            named_barrier(2, 256);
            if (tid == 0) {
                mbar_wait(bar(Plan::kBarGridOk), static_cast<uint32_t>(op & 1), flags);
                __threadfence();
                const unsigned old = atomicAdd(ch.sync + op, 1u);
                if (old == gridDim.x - 1) {
                    if (op > 0) ch.sync[op - 1] = 0;
                    if (op == n_ops - 1) ch.sync[op] = 0;
                }
            }
        }
        }  // op
    } else if (warp < kUMmaWarp + kUMmaWarps) {
        // =============================== MMA issuers ===============================
        // issuer `me` serves the decoder groups q with q % kNAcc == me and owns accumulator `me`
        // The whole warp runs the loop converged (so that addresses and descriptors stay in
        // uniform registers); one elected lane issues the tcgen05 instructions.
        const int wi = warp - kUMmaWarp;
        const int me = wi % NACC;  // accumulator (and decoder groups q % NACC == me) this warp serves
        const int tp = wi / NACC;  // which MMA tile of a group it issues when the tiles are split (TP == 2)
        const int t_lo = TP == 2 ? tp : 0, t_hi = TP == 2 ? tp + 1 : 2;
        if (wi < NACC * TP) {
            const bool leader = elect_one();
            uint32_t cnt0 = 0, cnt1 = 0, cnt2 = 0, cnt3 = 0;  // groups consumed from decoder group 0..3
            int segidx = 0, cbase = 0;  // segments / chunks of this CTA so far (all ops)
            int eg_base = 0;            // fp8: activation epochs of earlier ops
            for (int op = 0; op < n_ops; ++op) {
            const UmmaParams &p = ch.op[op];
            DMM_OP_GEOMETRY(p);
            // instruction descriptor: D fp32 (1) or int32 (2) at bit 4; A / B formats at bits 7 / 10
            // (f8f6f4: E2M3 = 3, E5M2 = 1; i8: signed = 1); N >> 3 at 17; M >> 4 at 24
            const uint32_t idesc = Pol::kIsInt
                                       ? ((2u << 4) | (1u << 7) | (1u << 10) | ((NMMA >> 3) << 17) | ((128u >> 4) << 24))
                                   : Pol::kIsF8
                                       ? ((1u << 4) | (3u << 7) | (1u << 10) | ((NMMA >> 3) << 17) | ((128u >> 4) << 24))
                                       : ((1u << 4) | ((NMMA >> 3) << 17) | ((128u >> 4) << 24));
            // descriptor of activation stage 0; later stages and k-halves only move the address field
            const uint32_t tile_b = plane_tile_bytes<NMMA, Pol::kIsInt != 0>(static_cast<int>(p.M));  // fp8: bytes of one k-tile of planes
            const int E = epoch_tiles(Plan::kEpochBytes, tile_b);  // k-tiles per epoch
            const int E0 = first_epoch_tiles(E, static_cast<int>(p.M), i1 - i0);  // the first one is short
            // fp8: a plane is one 8-row core matrix (rows past the batch overlap the next plane and
            // land in unused columns) or, for the 16-row layout, two of them
            const uint64_t xdesc0 = Pol::kIsF8 ? smem_desc(x_addr, tile_b / 2, (NMMA > 32 || Pol::kIsInt) ? 128u : tile_b / 8)
                                               : smem_desc(x_addr, NMMA * 16, 128);
            int cur_ep = -1, ep_beg = 0, ep_end = 0;  // fp8: epoch of this op being read and its k-tile range
            int ep_slot = eg_base % Plan::kEpochs;    // its buffer, the parity of that buffer's barriers
            uint32_t ep_par = static_cast<uint32_t>((eg_base / Plan::kEpochs) & 1), ep_addr = 0;
            const uint32_t xdesc_lo = static_cast<uint32_t>(xdesc0), xdesc_hi = static_cast<uint32_t>(xdesc0 >> 32);
            // accumulator of the (first) MMA tile this warp issues
            const uint32_t d_col0 = tmem + static_cast<uint32_t>(((TP == 2 ? tp : 0) * NACC + me) * NMMA);
            int jseg = 0;  // k-tiles of earlier segments of this op
            for (int ss = ss_first; ss <= ss_last; cbase += seg_chunks(ss), jseg += seg_len(ss), ++ss, ++segidx) {
                const int len = seg_len(ss);
                const int nchunks = (len + C - 1) / C;
                const int aset = segidx % Plan::kSets;  // accumulator set of this segment
                if (segidx >= Plan::kSets) {  // the epilogue has read what the set held before
                    mbar_wait(bar(Plan::kBarDFree + aset), static_cast<uint32_t>(((segidx / Plan::kSets) - 1) & 1), flags);
                    tc_fence_after();
                }
                [[maybe_unused]] const uint32_t d_seg = d_col0 + static_cast<uint32_t>(aset) * Plan::kSetCols;
                bool first = true;  // the accumulators hold nothing of this segment yet
                for (int c = (me - cbase) & (NACC - 1); c < nchunks; c += NACC) {
                    const int q = (cbase + c) & 3;
                    const int n = len - c * C < C ? len - c * C : C;
                    uint32_t cn = q == 0 ? cnt0 : q == 1 ? cnt1 : q == 2 ? cnt2 : cnt3;  // groups taken from group q so far
#pragma unroll 1
                    for (int g0 = 0; g0 < n; g0 += G, ++cn) {
                        const int sl = q * NA + static_cast<int>(cn % NA);
                        const uint32_t a_col = tmem + Plan::kDCols + static_cast<uint32_t>(sl) * Plan::kBufCols;
                        if constexpr (Pol::kIsF8) {
                            mbar_wait(bar(Plan::kBarFull + sl), (cn / NA) & 1, flags);
                            tc_fence_after();
                            // tile by tile (both MMA tiles of a k-tile back to back), so that an
                            // epoch is only left when nothing issued later still reads its buffer
#pragma unroll
                            for (int i = 0; i < G; ++i) {
                                if (g0 + i < n) {
                                    const int jt = jseg + c * C + g0 + i;  // CTA-wide k-tile index
                                    if (jt >= ep_end) {
                                        // step to the epoch that holds jt, releasing the ones left behind
                                        // (also epochs this issuer never read: every issuer arrives on
                                        // every epoch).  All state moves incrementally: no division, no
                                        // modulo in a loop that one thread runs between two MMAs.
                                        do {
                                            if (cur_ep >= 0) {
                                                if (leader) tc_commit(bar(Plan::kBarXFree + ep_slot));
                                                if (++ep_slot == Plan::kEpochs) {
                                                    ep_slot = 0;
                                                    ep_par ^= 1u;
                                                }
                                            }
                                            ++cur_ep;
                                            ep_beg = ep_end;
                                            ep_end += cur_ep == 0 ? E0 : E;
                                        } while (jt >= ep_end);
                                        mbar_wait(bar(Plan::kBarXReady + ep_slot), ep_par, flags);
                                        ep_addr = (static_cast<uint32_t>(ep_slot) * Plan::kEpochBytes) >> 4;
                                    }
                                    const uint32_t xlo = xdesc_lo + ep_addr + ((static_cast<uint32_t>(jt - ep_beg) * tile_b) >> 4);
                                    const uint32_t acc = (first && i == 0) ? 0u : 1u;
                                    if (leader) {
                                        if constexpr (TP == 1) {
                                            mma_ts_f8_lh<Pol::kIsInt != 0>(d_seg, a_col + i * Pol::kACols, xlo, xdesc_hi, idesc, acc);
                                            mma_ts_f8_lh<Pol::kIsInt != 0>(d_seg + NACC * NMMA, a_col + (G + i) * Pol::kACols, xlo, xdesc_hi, idesc, acc);
                                        } else {
                                            mma_ts_f8_lh<Pol::kIsInt != 0>(d_seg, a_col + (tp * G + i) * Pol::kACols, xlo, xdesc_hi, idesc, acc);
                                        }
                                    }
                                }
                            }
                        } else {
                            mbar_wait(bar(Plan::kBarFull + sl), (cn / NA) & 1, flags);
                            tc_fence_after();
                            const uint64_t xd = xdesc0 + ((static_cast<uint32_t>(sl) * Plan::kXStage) >> 4);
                            for (int t = t_lo; t < t_hi; ++t) {
                                const uint32_t d_col = tmem + static_cast<uint32_t>((t * NACC + me) * NMMA);
                                if (leader) {
                                    mma_ts_f16(d_col, a_col + t * G * Pol::kACols, xd, idesc, first ? 0u : 1u);
                                    mma_ts_f16(d_col, a_col + t * G * Pol::kACols + 8, xd + ((2 * NMMA * 16) >> 4), idesc, 1u);
                                }
                            }
                        }
                        first = false;
                        if (leader) tc_commit(bar(Plan::kBarFree + sl));
                    }
                    if (q == 0) cnt0 = cn; else if (q == 1) cnt1 = cn; else if (q == 2) cnt2 = cn; else cnt3 = cn;
                }
                if (leader) tc_commit(bar(Plan::kBarDReady + aset));
            }
            if constexpr (Pol::kIsF8) {
                const int nep = i1 <= i0 ? 0 : (i1 - i0 <= E0 ? 1 : 1 + (i1 - i0 - E0 + E - 1) / E);
                for (int r = cur_ep < 0 ? 0 : cur_ep; r < nep; ++r)
                    if (leader) tc_commit(bar(Plan::kBarXFree + (eg_base + r) % Plan::kEpochs));
                eg_base += nep;
                (void)ep_slot;
            }
            }  // op
        }
    } else if (warp >= kUTmaWarp) {
        // =============================== TMA producers ===============================
        // They stream the codes: chunk after chunk in the CTA-wide chunk order, each chunk one tiled load
        // (16 strips x C k-tiles) into the ring of the decoder group it belongs to.  Always the full box:
        // k-tiles past the segment are not used, strips past N read as zero.
        // Up to two batch rows four threads share the work, one per decoder group (four short independent
        // loops: a group whose ring is full does not hold up the others; measured 1 % faster at batch 1);
        // from three rows on one thread serves all groups in order (measured faster there).
        const int pw = warp - kUTmaWarp;
        constexpr bool split = kSplit;
        if (split) {
            const int q = pw;
            if (lane == 0) {
                const uint64_t policy = policy_evict_first();
                uint32_t n_q = 0;      // chunks issued for this group
                int slot = 0;          // n_q % RING
                uint32_t par = 1;      // parity of the Empty phase that frees `slot` (first pass: nothing to wait for)
                int cbase = 0;
                const UmmaParams &p = ch.op[0];
                DMM_OP_GEOMETRY(p);
                (void)p;
                for (int ss = ss_first; ss <= ss_last; cbase += seg_chunks(ss), ++ss) {
                    const int nchunks = seg_chunks(ss), kt0 = seg_kt0(ss);
                    for (int c = (q - cbase) & 3; c < nchunks; c += 4) {
                        if (n_q >= RING) mbar_wait(bar(Plan::kBarEmpty + q * RING + slot), par, flags);
                        const uint32_t b = bar(Plan::kBarCode + q * RING + slot);
                        mbar_arrive_expect_tx(b, Plan::kSlotBytes);
                        tma_load_2d(ring_addr + (q * RING + slot) * Plan::kSlotBytes, &ch.map[0], (kt0 + c * C) * (Pol::kFast ? 64 : 32), ss * (Pol::kFast ? 8 : 16), b, policy);
                        ++n_q;
                        if (++slot == RING) {
                            slot = 0;
                            par ^= 1u;
                        }
                    }
                }
                prefetch_next_codes(ch.op[0], cta, q, 4, 4 * RING * C);
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
        } else if (pw == 0) {
        if (lane == 0) {
            const uint64_t policy = policy_evict_first();
            uint32_t cnt[4] = {0, 0, 0, 0};  // chunks issued per decoder group
            int cbase = 0;
            for (int op = 0; op < n_ops; ++op) {
            const UmmaParams &p = ch.op[op];
            DMM_OP_GEOMETRY(p);
            (void)p;
            for (int ss = ss_first; ss <= ss_last; cbase += seg_chunks(ss), ++ss) {
                const int nchunks = seg_chunks(ss), kt0 = seg_kt0(ss);
                for (int c = 0; c < nchunks; ++c) {
                    const int q = (cbase + c) & 3;
                    const uint32_t n_q = q == 0 ? cnt[0] : q == 1 ? cnt[1] : q == 2 ? cnt[2] : cnt[3];
                    const int slot = static_cast<int>(n_q % RING);
                    if (n_q >= RING)
                        mbar_wait(bar(Plan::kBarEmpty + q * RING + slot), ((n_q / RING) - 1) & 1, flags);
                    const uint32_t b = bar(Plan::kBarCode + q * RING + slot);
                    mbar_arrive_expect_tx(b, Plan::kSlotBytes);
                    tma_load_2d(ring_addr + (q * RING + slot) * Plan::kSlotBytes, &ch.map[op], (kt0 + c * C) * (Pol::kFast ? 64 : 32), ss * (Pol::kFast ? 8 : 16), b, policy);
                    if (q == 0) ++cnt[0]; else if (q == 1) ++cnt[1]; else if (q == 2) ++cnt[2]; else ++cnt[3];
                }
            }
            }  // op
            prefetch_next_codes(ch.op[n_ops - 1], cta, 0, 1, 4 * RING * C);
            if (flags[0]) {
                // A wait gave up somewhere: loads may still be in flight.  Give the last load of
                // every ring slot a bounded chance to land before the CTA releases its shared memory.
                for (int q = 0; q < 4; ++q)
                    for (uint32_t d = 0; d < RING && d < cnt[q]; ++d) {
                        const uint32_t idx = cnt[q] - 1 - d;
                        mbar_wait_limit(bar(Plan::kBarCode + q * RING + static_cast<int>(idx % RING)), (idx / RING) & 1,
                                        20ll * 1000 * 1000);
                    }
            }
        }
        }
    } else {
        // =========================== activation loaders ===========================
        // loader wl serves the chunks of parity wl (the chunks of issuer wl), one chunk per pass
        // (a consumer of the slots form waits for the producer's flags instead, see below)
        if (!(kTp && p0.tp_mode == 3)) grid_dep_wait();
        const int wl = warp - kUMmaWarp - kUMmaWarps;  // warps 20 .. 23
        uint32_t cnt0 = 0, cnt1 = 0;  // fp16 policy: groups staged so far for decoder groups wl and wl + 2
        int cbase = 0;
        int eg_base = 0;              // fp8 policy: activation epochs of earlier ops
        for (int op = 0; op < n_ops; ++op) {
        const UmmaParams &p = ch.op[op];
        DMM_OP_GEOMETRY(p);
        if (n_ops > 1) {
            // Chain: op reads what op - 1 wrote, so wait until every CTA has finished op - 1
            // (bounded), then let this CTA's own arrival for op go ahead.
            if (op > 0) {
                if (lane == 0) grid_wait(ch.sync + (op - 1), gridDim.x, flags);
                __syncwarp();
            }
        }
        // Tensor-parallel consumer: wait (bounded) until every rank, this one included, has pushed the partial
        // product of the row-parallel layer before this one (epoch e, read in the prologue), then read the
        // activations as residual + all slots of that epoch's parity.  This wait stands in for the wait on the
        // previous kernel: this rank's own flag goes up only after every CTA of that kernel has finished, so
        // what it read may be cleared below and what it wrote is complete, and the kernels before it had
        // finished before it could.
        [[maybe_unused]] const float *tp_slots_now = nullptr;
        if (kTp && p.tp_mode == 3) {
            const unsigned e = static_cast<unsigned>(flags[3]);
            if (lane < p.tp_world) {
                const unsigned *mine = p.tp_flags[p.tp_rank] + lane;
                const long long t0 = clock64();
                for (;;) {
                    unsigned v;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
                    if (static_cast<int>(v - e) >= 0) break;
                    if (clock64() - t0 > p.tp_wait) {
                        raise_status(DMM_STATUS_WAIT_TIMEOUT);
                        break;
                    }
                    __nanosleep(40);
                }
            }
            __syncwarp();
            grid_dep_launch();
            tp_slots_now = p.peer_out[p.tp_rank] + static_cast<long long>(e & 1u) * p.tp_world * p.tp_count;
        }
        // a later kernel or op will accumulate into zero_ptr: clear it on the way -- in a chain before this
        // CTA's arrival for the op, otherwise after the activations are staged (nothing waits for it)
        auto clear_zero = [&]() {
            if (p.zero_ptr != nullptr) {
                constexpr int ZT = kULoadWarps * 32;
                for (long long i = static_cast<long long>(cta) * ZT + wl * 32 + lane; i < p.zero_count;
                     i += static_cast<long long>(gridDim.x) * ZT)
                    p.zero_ptr[i] = 0.f;
            }
        };
        if (n_ops > 1) clear_zero();
        if (kTp && p.tp_mode == 2) {
            // producer of epoch e + 1 (counter = e now that the previous kernel has finished): this rank's own
            // slot of parity e & 1 was read for the last time by the consumer before this kernel; clear it
            // for epoch e + 2
            constexpr int ZT = kULoadWarps * 32;
            const unsigned e = *reinterpret_cast<volatile const unsigned *>(p.tp_flags[p.tp_rank] + 16);
            float *z = p.peer_out[p.tp_rank] + (static_cast<long long>(e & 1u) * p.tp_world + p.tp_rank) * p.tp_count;
            for (long long i = static_cast<long long>(cta) * ZT + wl * 32 + lane; i < p.tp_count;
                 i += static_cast<long long>(gridDim.x) * ZT)
                z[i] = 0.f;
        }
        if (kTp && p.move_count > 0) {
            constexpr int ZT = kULoadWarps * 32;
            for (long long i = static_cast<long long>(cta) * ZT + wl * 32 + lane; i < p.move_count;
                 i += static_cast<long long>(gridDim.x) * ZT) {
                const float v = __ldcg(p.move_src + i);
                p.move_src[i] = 0.f;
                atomicAdd_system(p.move_dst + i, v);  // other ranks may already be adding their products (system scope, as theirs)
            }
        }
        if (n_ops > 1) {
            // the CTA's arrival for this op goes out only after this (so that it also covers the
            // clearing above, whatever share of the op's tiles this CTA has)
            __threadfence();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(Plan::kBarGridOk));
        }
        [[maybe_unused]] const __half *x = reinterpret_cast<const __half *>(p.x);
        const int M = static_cast<int>(p.M);
        const int ppt = M * 4;  // 16-byte pieces per k-tile: (row, 8-k chunk)

        if constexpr (Pol::kIsF8) {
            // The loaders never touch a barrier per tile: they fill whole epochs of the CTA's
            // k-tile sequence (segment after segment) with the four E5M2 planes of the activations,
            // densely packed [tile][k-half][plane][row][16 B]; the issuers point their operand
            // descriptors straight into these buffers.  A piece is 8 consecutive k of one row.
            constexpr int U = 4;  // pieces in flight per thread
            const uint32_t tile_b = plane_tile_bytes<NMMA, Pol::kIsInt != 0>(M);
            const int E = epoch_tiles(Plan::kEpochBytes, tile_b);
            // The first epoch is short: nothing can be multiplied before it is staged, and the
            // loaders may only start once the previous kernel of the stream has finished.
            const int E0 = first_epoch_tiles(E, M, i1 - i0);
            const int ntiles = i1 - i0;
            const int nep = ntiles <= 0 ? 0 : (ntiles <= E0 ? 1 : 1 + (ntiles - E0 + E - 1) / E);
            // two teams of loader warps fill alternate epochs, so that the global-memory latency
            // of one epoch overlaps the plane split of the other
            if (p.x_planes != nullptr && wl == 0 && lane == 0) {
                // The planes were split once by planes_kernel: an epoch is one bulk copy per
                // contiguous run of k-tiles (two when the CTA's tile sequence wraps to the next
                // super-tile inside the epoch).
                const uint8_t *src = reinterpret_cast<const uint8_t *>(p.x_planes);
                for (int e = 0; e < nep; ++e) {
                    const int eg = eg_base + e;  // epoch number over all ops: buffer and barrier phase
                    if (eg >= Plan::kEpochs)
                        mbar_wait(bar(Plan::kBarXFree + eg % Plan::kEpochs), static_cast<uint32_t>(((eg / Plan::kEpochs) - 1) & 1), flags);
                    const int t_lo = e == 0 ? 0 : E0 + (e - 1) * E;
                    const int e_len = e == 0 ? E0 : E;
                    const int nt = ntiles - t_lo < e_len ? ntiles - t_lo : e_len;
                    const uint32_t ebuf = x_addr + (eg % Plan::kEpochs) * Plan::kEpochBytes;
                    const uint32_t b = bar(Plan::kBarXReady + eg % Plan::kEpochs);
                    mbar_arrive_expect_tx(b, static_cast<uint32_t>(nt) * tile_b);
                    for (int t = 0; t < nt;) {
                        const int gt = i0 + t_lo + t;
                        const int kt = gt - (gt / KT) * KT;
                        const int run = KT - kt < nt - t ? KT - kt : nt - t;
                        bulk_g2s_plain(ebuf + t * tile_b, src + static_cast<size_t>(kt) * tile_b, static_cast<uint32_t>(run) * tile_b, b);
                        t += run;
                    }
                }
                if (flags[0]) {  // a wait gave up: let the copies in flight land before the CTA exits
                    for (int e = nep > Plan::kEpochs ? nep - Plan::kEpochs : 0; e < nep; ++e)
                        mbar_wait_limit(bar(Plan::kBarXReady + (eg_base + e) % Plan::kEpochs),
                                        static_cast<uint32_t>(((eg_base + e) / Plan::kEpochs) & 1), 20ll * 1000 * 1000);
                }
            }
            const int lt = (wl / kULoadTeams) * 32 + lane;
            constexpr int LT = kULoadWarps / kULoadTeams * 32;
            // (team by the epoch number over all ops, so that the teams keep alternating across ops)
            for (int e = ((wl % kULoadTeams) - eg_base) & (kULoadTeams - 1); p.x_planes == nullptr && e < nep; e += kULoadTeams) {
                const int eg = eg_base + e;
                if (eg >= Plan::kEpochs)
                    mbar_wait(bar(Plan::kBarXFree + eg % Plan::kEpochs), static_cast<uint32_t>(((eg / Plan::kEpochs) - 1) & 1), flags);
                const int t_lo = e == 0 ? 0 : E0 + (e - 1) * E;
                const int e_len = e == 0 ? E0 : E;
                const int nt = ntiles - t_lo < e_len ? ntiles - t_lo : e_len;
                const int npieces = nt * ppt;
                const uint32_t ebuf = x_addr + (eg % Plan::kEpochs) * Plan::kEpochBytes;
                if constexpr (Pol::kIsInt) {
                    // int8 activations go in as they are: a piece is 16 consecutive k of one row
                    const int8_t *x8 = reinterpret_cast<const int8_t *>(p.x);
                    const int nq = nt * 2 * M;
                    for (int pbase = 0; pbase < nq; pbase += LT * U) {
                        uint4 val[U];
                        uint32_t dst[U];
#pragma unroll
                        for (int u = 0; u < U; ++u) {
                            const int pc = pbase + u * LT + lt;
                            dst[u] = 0;
                            if (pc < nq) {
                                const int jl = pc / (2 * M), rem = pc - jl * (2 * M), row = rem >> 1, kh = rem & 1;
                                const int gt = i0 + t_lo + jl;
                                const int kt = gt - (gt / KT) * KT;
                                dst[u] = ebuf + jl * tile_b + kh * (tile_b / 2) + row * 16;
                                val[u] = __ldcg(reinterpret_cast<const uint4 *>(x8 + static_cast<long long>(row) * p.x_ld + 32 * kt + 16 * kh));
                            }
                        }
#pragma unroll
                        for (int u = 0; u < U; ++u)
                            if (dst[u] != 0) sts128(dst[u], val[u]);
                    }
                } else
                for (int pbase = 0; pbase < npieces; pbase += LT * U) {
                    uint32_t h[U][4];
                    uint32_t dst[U];
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        const int pc = pbase + u * LT + lt;
                        dst[u] = 0;
                        if (pc < npieces) {
                            const int jl = pc / ppt, rem = pc - jl * ppt, row = rem >> 2, kc = rem & 3;
                            const int gt = i0 + t_lo + jl;          // global tile index -> k-tile
                            const int kt = gt - (gt / KT) * KT;
                            const long long k0 = 32ll * kt + 8 * kc;
                            dst[u] = ebuf + jl * tile_b + (kc >> 1) * (tile_b / 2) + row * 16 + (kc & 1) * 8;
                            if (kTp && p.tp_mode == 3)
                                load_piece_sum(reinterpret_cast<const float *>(p.x), p.h_out, tp_slots_now, p.tp_world, p.tp_count, p.x_ld,
                                               row, k0, h[u]);
                            else
                                load_piece(p.x, p.x_mode, p.x_ld, p.x_gap, row, k0, h[u]);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < U; ++u) {
                        if (dst[u] != 0) {
#pragma unroll
                            for (int pl = 0; pl < 4; ++pl) {
                                const uint2 b8 = next_plane(h[u]);
                                sts64(dst[u] + pl * (tile_b / 8), b8.x, b8.y);
                            }
                        }
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(Plan::kBarXReady + eg % Plan::kEpochs));
            }
            eg_base += nep;
        } else {
            // fp16 activations: cp.async straight into the stage, two chunks in flight
            uint32_t pend_q[2] = {0, 0}, pend_cn[2] = {0, 0}, pend_ng[2] = {0, 0};
            int npend = 0;
            auto retire = [&]() {  // oldest pending chunk has landed
                fence_async_smem();
                __syncwarp();
                if (lane < static_cast<int>(pend_ng[0]))
                    mbar_arrive(bar(Plan::kBarFull + static_cast<int>(pend_q[0]) * NA + static_cast<int>((pend_cn[0] + lane) % NA)));
                pend_q[0] = pend_q[1]; pend_cn[0] = pend_cn[1]; pend_ng[0] = pend_ng[1];
                --npend;
            };
            // (two loader warps do this; the other two only work under the fp8 policy)
            for (int ss = ss_first; wl < 2 && ss <= ss_last; cbase += seg_chunks(ss), ++ss) {
                const int len = seg_len(ss), nchunks = seg_chunks(ss), kt0 = seg_kt0(ss);
                for (int c = (wl - cbase) & 1; c < nchunks; c += 2) {
                    const int q = (cbase + c) & 3;
                    const int n = len - c * C < C ? len - c * C : C;
                    const uint32_t cn = q < 2 ? cnt0 : cnt1;
                    const int ngroups = (n + G - 1) / G;
                    for (int gi = 0; gi < ngroups; ++gi) {
                        const uint32_t cg = cn + gi;
                        if (cg >= NA) mbar_wait(bar(Plan::kBarFree + q * NA + static_cast<int>(cg % NA)), ((cg / NA) - 1) & 1, flags);
                    }
                    for (int pc = lane; pc < n * ppt; pc += 32) {
                        const int i = pc / ppt, rem = pc - i * ppt, row = rem >> 2, kc = rem & 3;
                        const int sl = q * NA + static_cast<int>((cn + i / G) % NA);
                        cp_async16(x_addr + sl * Plan::kXStage + kc * (NMMA * 16) + row * 16,
                                   x + static_cast<long long>(row) * p.x_ld + 32 * (kt0 + c * C + i) + 8 * kc);
                    }
                    cp_async_commit();
                    pend_q[npend] = q; pend_cn[npend] = cn; pend_ng[npend] = ngroups;
                    ++npend;
                    if (q < 2) cnt0 += ngroups; else cnt1 += ngroups;
                    if (npend == 2) {
                        cp_async_wait<1>();
                        retire();
                    }
                }
            }
            while (npend > 0) {
                cp_async_wait<0>();
                retire();
            }
        }
        if (n_ops == 1) clear_zero();
        }  // op
    }

    tc_fence_before();
    __syncthreads();
    if (warp == kUMmaWarp) tmem_dealloc(tmem, kUTmemCols);
}

// L2 prefetch of the first `tiles` k-tiles (at most) that CTA `cta` of the next launch will stream: for each
// of the 16 strips of its first super-tile one contiguous run of the strip's code stream.  `part` of the
// strips (part of 4) is done by the caller, so that four producer threads can share the work.
__device__ __forceinline__ void prefetch_next_codes(const UmmaParams &p, int cta, int part, int nparts, int tiles) {
    if (p.next_codes == nullptr || cta >= p.next_grid) return;
    const int KT = static_cast<int>(p.next_K / 32);
    const int i0 = part32_begin(p.next_part, cta), i1 = part32_begin(p.next_part, cta + 1);
    const int ss = i0 / KT, kt0 = i0 - ss * KT;
    int n = i1 - i0 < tiles ? i1 - i0 : tiles;
    if (n > KT - kt0) n = KT - kt0;  // (a range that wraps into the next super-tile: its first part only)
    if (n <= 0) return;
    const long long strips = p.next_N / 16;
    const uint8_t *base = reinterpret_cast<const uint8_t *>(p.next_codes);
    for (int s = part; s < 16; s += nparts) {
        const long long strip = static_cast<long long>(ss) * 16 + s;
        if (strip >= strips) break;
        const uint8_t *src = base + (strip * KT + kt0) * 128;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(static_cast<uint32_t>(n) * 128u) : "memory");
    }
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link-time libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

// Tensor map of the tiled code matrix seen as uint32 [strips][K/32 * 32], box = c_tiles k-tiles x 16 strips.
// With `fast` the matrix is in the layout of fast_decode_matmul_cuda, seen as uint32 [row blocks of 32][K/16 * 32]:
// a k-tile of a row block is 64 consecutive words, box = c_tiles k-tiles x 8 row blocks (the same 8 KiB).
inline int make_codes_map(CUtensorMap *map, const void *codes, long long N, long long K, int c_tiles, bool fast = false) {
    // A model calls with the same weight matrices over and over: the maps a host thread has encoded are kept
    // (a map depends on nothing but these arguments, so a recycled address gives the same map).
    struct Key {
        const void *codes;
        long long N, K;
        int c_tiles, fast;
        bool operator==(const Key &o) const { return codes == o.codes && N == o.N && K == o.K && c_tiles == o.c_tiles && fast == o.fast; }
    };
    struct KeyHash {
        size_t operator()(const Key &k) const {
            return std::hash<const void *>()(k.codes) ^ (static_cast<size_t>(k.N) * 0x9E3779B97F4A7C15ull) ^ (static_cast<size_t>(k.K) << 20) ^
                   static_cast<size_t>(k.c_tiles * 2 + k.fast);
        }
    };
    thread_local std::unordered_map<Key, CUtensorMap, KeyHash> cache;
    const Key key{codes, N, K, c_tiles, fast ? 1 : 0};
    const auto hit = cache.find(key);
    if (hit != cache.end()) {
        *map = hit->second;
        return 0;
    }
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return cudaErrorNotSupported;
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(fast ? 2 * K : K), static_cast<cuuint64_t>(fast ? N / 32 : N / 16)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(K) * (fast ? 8 : 4)};  // bytes per strip / row block
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(c_tiles * (fast ? 64 : 32)), static_cast<cuuint32_t>(fast ? 8 : 16)};
    const cuuint32_t estride[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(codes), gdim, gstride, box, estride,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    if (cache.size() >= 8192) cache.clear();  // (bounded: a process that streams ever new matrices just re-encodes)
    cache.emplace(key, *map);
    return 0;
}

template <class Pol, int NMMA, bool kChain>
inline int launch_umma_ops(const UmmaParams *ops, int n_ops, unsigned *sync, int num_sms, bool pdl, cudaStream_t stream);

// Launches `n_ops` products as one kernel.  n_ops == 1 (kChain false): the plain case, grid =
// min(tiles, SMs).  A chain (kChain true): grid = SMs for every op and a cooperative launch, because
// the CTAs wait for one another between ops and must all be resident; `sync` = n_ops zeroed counters.
template <class Pol, int NMMA, bool kChain>
inline int launch_umma_ops(const UmmaParams *ops, int n_ops, unsigned *sync, int num_sms, bool pdl, cudaStream_t stream) {
    using Plan = UmmaPlan<Pol, NMMA>;
    auto kernel = umma_kernel<Pol, NMMA, kChain, false>;
    // four TMA producer warps up to two batch rows of the fp16 family (measured 1 % faster at batch 1), else one
    bool split = false;
    [[maybe_unused]] const bool tp_variant = ops[0].n_peers > 0 || ops[0].move_count > 0 || ops[0].tp_mode != 0;
    if constexpr (Pol::kIsF8 && !kChain && !Pol::kFast) {  // tensor-parallel epilogue: its own instantiation, nothing of it in the plain kernel
        if (tp_variant) kernel = umma_kernel<Pol, NMMA, kChain, true>;
    }
    if constexpr (Pol::kIsF8 && !Pol::kIsInt && !kChain && NMMA == 16 && !Pol::kFast) {
        if (ops[0].M <= 2) {
            split = true;
            kernel = umma_kernel<Pol, NMMA, kChain, false, true>;
            if (ops[0].n_peers > 0 || ops[0].move_count > 0 || ops[0].tp_mode != 0) kernel = umma_kernel<Pol, NMMA, kChain, true, true>;
        }
    }
    // the shared-memory attribute is set once per kernel variant and device, not on every launch
    static std::atomic<unsigned long long> attr_done[4];
    const int variant = (tp_variant ? 1 : 0) | (split ? 2 : 0);
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev >= 64 || !((attr_done[variant].load(std::memory_order_acquire) >> dev) & 1ull)) {
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Plan::kDynBytes));
        if (err != cudaSuccess) return err;
        if (dev < 64) attr_done[variant].fetch_or(1ull << dev, std::memory_order_release);
    }
    UmmaChainT<kChain ? kMaxOps : 1> ch = {};
    ch.n_ops = n_ops;
    ch.sync = sync;
    unsigned grid = static_cast<unsigned>(num_sms);
    if (!kChain) {
        const long long T = ((ops[0].N / 16 + 15) / 16) * (ops[0].K / 32);
        if (T < num_sms) grid = static_cast<unsigned>(T);
    }
    for (int i = 0; i < n_ops; ++i) {
        UmmaParams &p = ch.op[i];
        p = ops[i];
        p.dyn_smem_bytes = Plan::kDynBytes;
        const long long KT = p.K / 32, NS = p.N / 16, SST = (NS + 15) / 16;
        const long long T = SST * KT;
        if (T >= (1ll << 31)) return DMM_ERR_SHAPE;
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
        if (Pol::kFast) p.next_codes = nullptr;  // (the prefetch hint describes the tile layout)
        if ((p.fast_layout != 0) != (Pol::kFast != 0)) return DMM_ERR_ARG;
        const int rc = make_codes_map(&ch.map[i], p.codes, p.N, p.K, Pol::kC, Pol::kFast != 0);
        if (rc) return rc;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(split ? kUThreads : kUThreads - (kUTmaWarps - 1) * 32);
    cfg.dynamicSmemBytes = Plan::kDynBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (kChain) {
        attr[na].id = cudaLaunchAttributeCooperative;
        attr[na].val.cooperative = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kernel, ch);
}

template <class Pol, int NMMA>
inline int launch_umma_one(const UmmaParams &p, int num_sms, bool pdl, cudaStream_t stream) {
    return launch_umma_ops<Pol, NMMA, false>(&p, 1, nullptr, num_sms, pdl, stream);
}

// A chain of up to kMaxOps dependent products, batch <= 8 (fp8 policy, activations split in the kernel).
inline int launch_umma_chain(const UmmaParams *ops, int n_ops, unsigned *sync, int num_sms, bool pdl, cudaStream_t stream) {
    if (n_ops < 2 || n_ops > kMaxOps) return DMM_ERR_ARG;
    return launch_umma_ops<PolF8, 32, true>(ops, n_ops, sync, num_sms, pdl, stream);
}

// From this batch size on the fp8-operand path splits the activations into planes with
// planes_kernel before the matmul kernel instead of inside it.
constexpr long long kPlanesMinBatch = 4;

// Padded batch rows of the plane layout for a batch of M (<= 32) rows.
inline int planes_rows(long long M) { return M <= 8 ? static_cast<int>(M) : (M <= 16 ? 16 : 32); }

inline int launch_planes(const void *x, int x_mode, long long x_ld, long long x_gap, int M, long long K, uint8_t *planes,
                         bool pdl, cudaStream_t stream) {
    const long long pieces = K / 16 * 2 * M;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>((pieces + 127) / 128));
    cfg.blockDim = dim3(128);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, planes_kernel, x, x_mode, x_ld, x_gap, M, K, planes_rows(M), planes);
}

// Integer family: int8 activations, up to 32 batch rows per launch, int32 result.
inline int launch_umma_i8(const UmmaParams &p, int num_sms, bool pdl, cudaStream_t stream) {
    if (p.fast_layout) {
        if (p.M <= 16) return launch_umma_one<PolI8Fast, 16>(p, num_sms, pdl, stream);
        return launch_umma_one<PolI8Fast, 32>(p, num_sms, pdl, stream);
    }
    if (p.M <= 16) return launch_umma_one<PolI8, 16>(p, num_sms, pdl, stream);
    return launch_umma_one<PolI8, 32>(p, num_sms, pdl, stream);
}

// f8 != 0: PolF8 (needs M <= 32); else PolF16 with M <= 64.
inline int launch_umma(bool f8, const UmmaParams &p, int num_sms, bool pdl, cudaStream_t stream) {
    if (f8 && p.fast_layout) {
        if (p.M <= 8) return launch_umma_one<PolF8Fast, 32>(p, num_sms, pdl, stream);
        if (p.M <= 16) return launch_umma_one<PolF8Fast, 64>(p, num_sms, pdl, stream);
        return launch_umma_one<PolF8Fast, 128>(p, num_sms, pdl, stream);
    }
    if (f8) {
        // up to two batch rows all four planes fit one 8-row core matrix: 16 MMA columns instead of 32 halve
        // what the tensor core reads from shared memory per MMA (the build with four TMA producers).  For 3
        // and 4 rows (two core matrices of the dense planes) it measured 1-2 % faster but cost batch 2 3 %.
        if (p.M <= 2) return launch_umma_one<PolF8, 16>(p, num_sms, pdl, stream);
        if (p.M <= 8) return launch_umma_one<PolF8, 32>(p, num_sms, pdl, stream);
        if (p.M <= 16) return launch_umma_one<PolF8, 64>(p, num_sms, pdl, stream);
        return launch_umma_one<PolF8, 128>(p, num_sms, pdl, stream);
    }
    if (p.M <= 16) return launch_umma_one<PolF16, 16>(p, num_sms, pdl, stream);
    if (p.M <= 32) return launch_umma_one<PolF16, 32>(p, num_sms, pdl, stream);
    return launch_umma_one<PolF16, 64>(p, num_sms, pdl, stream);
}

// Workspace floats per CTA slot for a batch of M columns on this path.
inline int umma_partial_values(long long M, bool f8) {
    const int nb = f8 ? (M <= 8 ? 8 : (M <= 16 ? 16 : 32)) : (M <= 16 ? 16 : (M <= 32 ? 32 : 64));
    return 2 * nb * 128;
}

}  // namespace dmm
