// Shared device helpers: PTX wrappers, the replicated decode table and the decode core.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dmm.h"

namespace dmm {

// ---------------------------------------------------------------------------------------
// Device status word (one per device that loads the library).  Kernels OR bits into it;
// dmm_status() reads and clears it.  The library is built as a single translation unit
// (dmm_api.cu includes every kernel header), so this is the only definition.
// ---------------------------------------------------------------------------------------
__device__ unsigned g_status = 0;

__device__ __forceinline__ void raise_status(unsigned bits) { atomicOr(&g_status, bits); }

// ---------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// try_wait that lets the hardware keep the thread suspended for up to `hint_ns` while the phase
// is pending (it resumes as soon as the phase completes): a waiting warp then issues next to
// nothing and leaves its scheduler to the warps that have work.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}

// Waits for a phase of an mbarrier, but never for longer than about a quarter of a second:
// on expiry the CTA-wide `failed` flag is set, the device status word gets
// DMM_STATUS_WAIT_TIMEOUT and every later wait of the CTA returns at once, so a lost
// arrival produces a wrong result with a raised status instead of a hung GPU.
constexpr long long kWaitLimitCycles = 500ll * 1000 * 1000;
constexpr uint32_t kWaitHintNs = 20000;  // longest single suspension inside a wait

__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int *failed) {
    if (mbar_try_wait(bar, parity)) return;
    if (*failed) return;
    const long long t0 = clock64();
    for (;;) {
        // try_wait suspends the thread for a hardware-defined while: poll a few times between
        // looks at the clock so that a waiting warp costs almost no issue slots
#pragma unroll 1
        for (int i = 0; i < 16; ++i)
            if (mbar_try_wait_hint(bar, parity, kWaitHintNs)) return;
        if (clock64() - t0 > kWaitLimitCycles || *failed) {
            if (!*failed) {
                *failed = 1;
                raise_status(DMM_STATUS_WAIT_TIMEOUT);
            }
            return;
        }
    }
}

// Waits (bounded, like mbar_wait) until a counter in global memory that other CTAs of the same
// grid increment has reached `target`.  Only legal when all those CTAs are resident together.
__device__ __forceinline__ void grid_wait(const unsigned *counter, unsigned target, volatile int *failed) {
    if (*failed) return;
    const long long t0 = clock64();
    for (;;) {
        unsigned v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if (v >= target) return;
        if (clock64() - t0 > kWaitLimitCycles || *failed) {
            if (!*failed) {
                *failed = 1;
                raise_status(DMM_STATUS_WAIT_TIMEOUT);
            }
            return;
        }
        __nanosleep(40);
    }
}

// A plain bounded wait that ignores the CTA's failed flag: used on the way out of a kernel whose
// earlier wait gave up, to let copies that are still in flight land.
__device__ __forceinline__ void mbar_wait_limit(uint32_t bar, uint32_t parity, long long cycles) {
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > cycles) return;
    }
}

// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
// dst, src and bytes must be multiples of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes,
                                         uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}

// The same without a cache hint (data that other CTAs read again from L2).
__device__ __forceinline__ void bulk_g2s_plain(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// 2-D tiled TMA load (tensor map in kernel parameter space), completion counted on an mbarrier.
// x is in elements of the map's data type and x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, int x, int y, uint32_t bar,
                                            uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
        "l"(tmap), "r"(x), "r"(y), "r"(bar), "l"(policy)
        : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// arrives at a named barrier without waiting for it
__device__ __forceinline__ void named_barrier_arrive(int id, int threads) {
    __threadfence_block();
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------------------------------
// Decode table in shared memory.
//
// 256 rows of 256 bytes at a 64 KiB-aligned shared address.  Row e holds
//   bytes   0..127 : codebook entry e (8 x int8 = 4*value), replicated 16 times
//   bytes 128..255 : sign/shift mask for high code byte e, replicated 16 times
// Lane l reads replica l % 16, so a warp-wide 8-byte load is conflict free whatever the
// indices are, and because row addresses are (index << 8) one byte-permute builds the
// address from a code word.
//
// The decode itself is two XORs.  For a table byte v with low bits "10":
//   -v == v ^ 0xFC,  v + 1 == v ^ 0x01,  v - 1 == v ^ 0x03
// (the identity behind decode8weights, decode_matmul_cuda.cu:58-62), so
//   decoded = entry[code & 0xFF] ^ mask[code >> 8]
// with mask byte i = (sign_i ? 0xFC : 0) ^ (shift ? 0x03 : 0x01) ^ extra, where extra is 0
// for the integer family and 0x80 (offset binary) for the fp16 family.  A third byte format
// (sign-magnitude, for fp6 tensor-core operands) obeys the same entry ^ mask rule.
// ---------------------------------------------------------------------------------------
constexpr uint32_t kLutBytes = 65536;

// Byte formats the table can produce (the XOR of an entry and a mask byte):
//   kFmtTwos    two's complement int8 q                (integer family, legacy MMA)
//   kFmtOffset  offset binary q + 128                  (fp16 family: 0x6400|u is the half 1024+u)
//   kFmtFp6     sign << 5 | |q|, |q| <= 15             (fp6 E2M3 container: the value is q/8,
//               because E2M3 codes 0..15 are linear: exponent 0 is subnormal m/8, exponent 1 is
//               (8+m)/8)
constexpr int kFmtTwos = 0, kFmtOffset = 1, kFmtFp6 = 2;

// Mask bytes for high code byte h (bit 7 = shift, bits 0..6 = stored signs).
__host__ __device__ inline uint64_t sign_mask(uint32_t h, int convention, int fmt) {
    const uint32_t s7 = h & 0x7Fu;
    uint32_t par = s7;
    par ^= par >> 4;
    par ^= par >> 2;
    par ^= par >> 1;
    par &= 1u;
    const uint32_t s8 = convention == DMM_SIGN_SLOW ? (s7 | (par << 7)) : ((s7 << 1) | par);
    const uint32_t shift = (h >> 7) & 1u;
    uint64_t m = 0;
    for (int i = 0; i < 8; ++i) {
        const uint32_t sg = (s8 >> i) & 1u;
        uint64_t b;
        if (fmt == kFmtFp6) {
            b = (sg << 5) | ((sg ^ shift) << 1);
        } else {
            b = (sg ? 0xFCu : 0x00u) ^ (shift ? 0x03u : 0x01u) ^ (fmt == kFmtOffset ? 0x80u : 0x00u);
        }
        m |= b << (8 * i);
    }
    return m;
}

// kFmtFp6 masks carry two bits per weight, so they are stored as ONE 32-bit word per high
// byte: weights 0..3 at bits 8j+1 (sign ^ shift) and 8j+5 (sign), weights 4..7 one bit
// lower.  (word & 0x22222222) and ((word << 1) & 0x22222222) are the two byte-mask words.
// A 4-byte look-up is one shared-memory wavefront per warp instead of two.
__host__ __device__ inline uint32_t sign_mask_fp6_packed(uint32_t h, int convention) {
    const uint64_t m = sign_mask(h, convention, kFmtFp6);
    const uint32_t lo = static_cast<uint32_t>(m), hi = static_cast<uint32_t>(m >> 32);
    return (lo & 0x22222222u) | ((hi & 0x22222222u) >> 1);
}

// Codebook entry e as packed int8 x 8 (= 4 * value), from either table format.  Sets *bad
// when the entry cannot be decoded by XOR (byte not congruent to 2 mod 4, fp16 value not k/4).
__device__ inline uint64_t load_entry(const void *cb, int cb_is_f16, int e, bool *bad, const uint4 *pre = nullptr) {
    uint64_t v;
    if (!cb_is_f16) {
        v = static_cast<uint64_t>(reinterpret_cast<const int64_t *>(cb)[e]);
    } else {
        const uint4 raw = pre != nullptr ? *pre : reinterpret_cast<const uint4 *>(cb)[e];
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        v = 0;
        for (int i = 0; i < 8; ++i) {
            const __half h = __ushort_as_half(static_cast<unsigned short>((w[i >> 1] >> (16 * (i & 1))) & 0xFFFFu));
            const float f = __half2float(h) * 4.0f;
            const int q = __float2int_rn(f);
            if (!(static_cast<float>(q) == f) || q < -127 || q > 127) *bad = true;
            v |= static_cast<uint64_t>(static_cast<uint32_t>(q) & 0xFFu) << (8 * i);
        }
    }
    if (((v & 0x0303030303030303ull) ^ 0x0202020202020202ull) != 0) *bad = true;
    return v;
}

// Entry bytes in the given format.  kFmtFp6: (neg << 5) | ((|c| | 1) ^ (neg << 1)); XOR with
// the mask byte gives sign = s ^ neg and magnitude |c| + 1 or |c| - 1.
__device__ inline uint64_t format_entry(uint64_t v, int fmt, bool *bad) {
    if (fmt != kFmtFp6) return v;
    uint64_t r = 0;
    for (int i = 0; i < 8; ++i) {
        const int c = static_cast<int8_t>((v >> (8 * i)) & 0xFFu);
        const uint32_t neg = c < 0 ? 1u : 0u;
        const uint32_t mag = static_cast<uint32_t>(c < 0 ? -c : c);
        if (mag > 14u) *bad = true;
        r |= static_cast<uint64_t>((neg << 5) | (((mag | 1u) ^ (neg << 1)) & 0x1Fu)) << (8 * i);
    }
    return r;
}

// Fills the table; every thread of the group calls it (tid in [0, nthreads)).
// Returns true when this thread saw an entry that the XOR decode cannot represent.
// packed_mask: store the kFmtFp6 masks as 32 replicas of the packed 32-bit word.
// Work item i < 512: entry row i & 255, half i >> 8 (0 = table entry, 1 = sign mask), so that the
// lanes of a warp all take the same branch.
// pre: the fp16 entry of thread tid (tid < 256), loaded earlier with lut_prefetch so that
// the global-memory latency overlaps other set-up work (needs nthreads >= 512).
__device__ __forceinline__ uint4 lut_prefetch(const void *cb16, int tid) {
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tid < 256) v = __ldg(reinterpret_cast<const uint4 *>(cb16) + tid);
    return v;
}

__device__ inline bool lut_fill(uint32_t lut_addr, const void *cb, int cb_is_f16, int convention,
                                int fmt, int tid, int nthreads, bool packed_mask = false, const uint4 *pre = nullptr) {
    bool bad = false;
    for (int i = tid; i < 512; i += nthreads) {
        const int e = i & 255;
        const int part = i >> 8;
        uint4 rep;
        if (part == 1 && packed_mask) {
            const uint32_t w = sign_mask_fp6_packed(static_cast<uint32_t>(e), convention);
            rep = make_uint4(w, w, w, w);
        } else {
            const uint64_t v = part == 0 ? format_entry(load_entry(cb, cb_is_f16, e, &bad, pre), fmt, &bad)
                                         : sign_mask(static_cast<uint32_t>(e), convention, fmt);
            const uint32_t lo = static_cast<uint32_t>(v), hi = static_cast<uint32_t>(v >> 32);
            rep = make_uint4(lo, hi, lo, hi);
        }
        const uint32_t base = lut_addr + static_cast<uint32_t>(e) * 256u + static_cast<uint32_t>(part) * 128u;
        // Consecutive threads own consecutive 128-byte half rows (same banks): start each at a
        // different 16-byte chunk so that a warp-wide store touches every bank equally.
#pragma unroll
        for (int r = 0; r < 8; ++r) sts128(base + 16u * static_cast<uint32_t>((r + i) & 7), rep);
    }
    return bad;
}

// Per-lane constants for the byte-permute address build: byte 0 = replica offset (+128 for
// the mask half of a row), bytes 2..3 = the table's 64 KiB-aligned shared address.
struct LutLane {
    uint32_t entry_c;  // lut_addr | (lane%16)*8
    uint32_t mask_c;   // lut_addr | 128 | (lane%16)*8, or | lane*4 for packed masks
    uint32_t two;      // the number 2 in a register the compiler cannot see through (keeps a multiply a multiply)
};

__device__ __forceinline__ LutLane lut_lane(uint32_t lut_addr, int lane, bool packed_mask = false) {
    LutLane l;
    l.entry_c = lut_addr | (static_cast<uint32_t>(lane & 15) << 3);
    l.mask_c = packed_mask ? (lut_addr | 128u | (static_cast<uint32_t>(lane) << 2)) : (l.entry_c | 128u);
    l.two = 2u;
    return l;
}

// kFmtFp6 with packed masks: 8-byte entry look-up, 4-byte mask look-up, two XORs.
template <int which>
__device__ __forceinline__ uint2 decode8_fp6(uint32_t word, const LutLane &l) {
    constexpr uint32_t sel_idx = which == 0 ? 0x7604u : 0x7624u;
    constexpr uint32_t sel_hi = which == 0 ? 0x7614u : 0x7634u;
    const uint2 e = lds64(prmt(word, l.entry_c, sel_idx));
    const uint32_t m = lds32(prmt(word, l.mask_c, sel_hi));
    uint32_t m2;  // m << 1 as an integer multiply-add: the FMA pipe is idle, the integer ALU is not
    asm("mad.lo.u32 %0, %1, %2, 0;" : "=r"(m2) : "r"(m), "r"(l.two));
    return make_uint2(e.x ^ (m & 0x22222222u), e.y ^ (m2 & 0x22222222u));
}

// Decodes the code in half `which` (0 = low 16 bits, 1 = high) of `word`: 8 packed bytes.
template <int which>
__device__ __forceinline__ uint2 decode8(uint32_t word, const LutLane &l) {
    // result bytes: [const byte0, selected code byte, const byte2, const byte3]
    constexpr uint32_t sel_idx = which == 0 ? 0x7604u : 0x7624u;
    constexpr uint32_t sel_hi = which == 0 ? 0x7614u : 0x7634u;
    const uint2 e = lds64(prmt(word, l.entry_c, sel_idx));
    const uint2 m = lds64(prmt(word, l.mask_c, sel_hi));
    return make_uint2(e.x ^ m.x, e.y ^ m.y);
}

// Offset-binary bytes (q + 128) -> fp16 pairs holding the integers q exactly:
// 0x6400 | u is the half 1024 + u, and subtracting 1152 leaves q.
__device__ __forceinline__ void bytes_to_half2(uint2 d, uint32_t (&r)[4]) {
    const __half2 bias = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));
    const uint32_t magic = 0x64646464u;
    uint32_t t[4] = {prmt(d.x, magic, 0x4140u), prmt(d.x, magic, 0x4342u), prmt(d.y, magic, 0x4140u),
                     prmt(d.y, magic, 0x4342u)};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = *reinterpret_cast<__half2 *>(&t[i]);
        h = __hsub2(h, bias);
        r[i] = *reinterpret_cast<uint32_t *>(&h);
    }
}

// ---------------------------------------------------------------------------------------
// Balanced partition of T work items over G CTAs in 32-bit arithmetic (T < 2^31):
// with a = T / G and b = T % G (computed on the host), the first b CTAs own a + 1 items.
// ---------------------------------------------------------------------------------------
struct Part32 {
    int a, b;
};
__host__ __device__ inline int part32_begin(Part32 pt, int c) { return pt.a * c + (c < pt.b ? c : pt.b); }
__host__ __device__ inline int part32_owner(Part32 pt, int i) {
    const int big = pt.b * (pt.a + 1);
    return i < big ? i / (pt.a + 1) : pt.b + (i - big) / pt.a;
}

// ---------------------------------------------------------------------------------------
// Stream-K partition of T work items over G CTAs: CTA c owns [T*c/G, T*(c+1)/G).
// ---------------------------------------------------------------------------------------
__host__ __device__ inline long long part_begin(long long T, long long G, long long c) { return T * c / G; }
// The CTA whose range contains item i.
__host__ __device__ inline long long part_owner(long long T, long long G, long long i) {
    return ((i + 1) * G - 1) / T;
}

}  // namespace dmm
