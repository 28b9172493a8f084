// Decode-core micro-benchmark (a standalone program, not part of libdmm.so): how many cycles per 2 KiB tile
// (1024 codes = 256 rows x 32 k) can one SM sustain for code fetch + table look-ups + XOR + tcgen05.st, with no
// MMA, no TMA and no hand-over between warps?  The answer is the floor that the decode puts under the small-batch
// kernel, and it compares the decodes that were candidates for it.  Build and run (one B200, a few seconds):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o decode_core_bench decode_matmul_b200/csrc/decode_core_bench.cu
//   ./decode_core_bench
// Every CTA runs 16..32 decoder warps in groups of four over codes resident in shared memory; the table contents
// are arbitrary (timing does not depend on the values), so nothing here is checked for correctness.
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include "dmm_common.cuh"
#include "dmm_umma.cuh"
using namespace dmm;

// VAR bits: 1 = mask shift as a multiply-add (FMA pipe) instead of a funnel shift (ALU pipe);
//           2 = no tcgen05.st (XOR into a sink);  4 = codes through tcgen05.ld instead of lds.128;
//           8 = mbarrier arrive + tcgen05 fences per step;
//          16 = 4-byte entries of eight nibbles (one lds.32, expanded with two masks and a shift) instead of
//               8-byte entries
template <int VAR, int G>
__global__ void __launch_bounds__(1024, 1) k(uint32_t *out, int iters, long long *cyc) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t lut_addr = (base + 2048 + 0xFFFFu) & ~0xFFFFu;
    const uint32_t code_addr = lut_addr + kLutBytes;  // 32 KB of codes: 4 slots of [16 strips][4 k-tiles][128 B]
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) uint64_t bars[8];
    const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
    const int nwarps = blockDim.x >> 5;
    // table: any contents; fill pseudo-randomly (timing does not depend on the values)
    for (uint32_t o = tid * 16u; o < kLutBytes + 32768u; o += blockDim.x * 16u) {
        uint32_t s = o * 2654435761u + blockIdx.x;
        sts128(lut_addr + o, make_uint4(s, s * 3u, s * 5u, s * 7u));
    }
    if (tid < 8) mbar_init(smem_u32(&bars[tid]), 4);
    fence_mbar_init();
    if (warp == 0) tmem_alloc(smem_u32(&tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    const int q = warp >> 2, wq = warp & 3;
    const LutLane ll = lut_lane(lut_addr, lane, true);
    const uint32_t tlane = tmem + (static_cast<uint32_t>(wq * 32) << 16);
    const uint32_t colbase = tlane + static_cast<uint32_t>(q) * 64;  // 64 columns per group (up to 8 groups)
    if (VAR & 4) {  // park codes in TMEM columns q*64+48.. (16 columns = 4 k-tiles)
        uint32_t r[16];
        for (int i = 0; i < 16; ++i) r[i] = lds32(code_addr + ((tid * 16 + i) * 4 & 32767));
        tmem_st16(colbase + 48, r);
        tmem_wait_st();
    }
    __syncthreads();
    const long long t0 = clock64();
    uint32_t sink = 0;
    const uint32_t src0 = code_addr + (wq * 4 + (lane >> 3)) * 512 + (lane & 7) * 16;
#pragma unroll 1
    for (int it = 0; it < iters; ++it) {
        const uint32_t src = src0 + ((it + q) & 3) * 8192;
#pragma unroll
        for (int g2 = 0; g2 < G; g2 += 2) {
            uint32_t r0[16], r1[16];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                uint4 cw;
                if (VAR & 4) {
                    uint32_t t4[4];
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(t4[0]), "=r"(t4[1]), "=r"(t4[2]), "=r"(t4[3])
                                 : "r"(colbase + 48 + ((g2 + i) & 3) * 4)
                                 : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(t4[0]), "+r"(t4[1]), "+r"(t4[2]), "+r"(t4[3])::"memory");
                    cw = make_uint4(t4[0] + it, t4[1], t4[2], t4[3]);
                } else {
                    cw = lds128(src + ((g2 + i) & 3) * 128);
                }
                const uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    uint2 d0, d1;
                    if (VAR & 16) {
                        // entry word: byte k = nibble of weight k (low) and of weight k + 4 (high), nibble = [t1 t0 0 1];
                        // mask word: bits 8k+1 / 8k+5 for weights k (sign^shift, sign), 8k+0 / 8k+4 for weights k + 4
                        const uint32_t e0 = lds32(prmt(w[t], ll.mask_c, 0x7604u));
                        const uint32_t m0 = lds32(prmt(w[t], ll.mask_c, 0x7614u));
                        const uint32_t e1 = lds32(prmt(w[t], ll.mask_c, 0x7624u));
                        const uint32_t m1 = lds32(prmt(w[t], ll.mask_c, 0x7634u));
                        uint32_t m0s, m1s, e0s, e1s;
                        asm("mad.lo.u32 %0, %1, 2, 0;" : "=r"(m0s) : "r"(m0));
                        asm("mad.lo.u32 %0, %1, 2, 0;" : "=r"(m1s) : "r"(m1));
                        asm("mul.hi.u32 %0, %1, 0x10000000;" : "=r"(e0s) : "r"(e0));  // e >> 4 on the FMA pipe
                        asm("mul.hi.u32 %0, %1, 0x10000000;" : "=r"(e1s) : "r"(e1));
                        // lo = (e & 0x0F0F0F0F) ^ (m & 0x22222222): two ops (a 4-input function); hi likewise
                        d0 = make_uint2((e0 & 0x0F0F0F0Fu) ^ (m0 & 0x22222222u), (e0s & 0x0F0F0F0Fu) ^ (m0s & 0x22222222u));
                        d1 = make_uint2((e1 & 0x0F0F0F0Fu) ^ (m1 & 0x22222222u), (e1s & 0x0F0F0F0Fu) ^ (m1s & 0x22222222u));
                    } else if (VAR & 1) {
                        const uint2 e0 = lds64(prmt(w[t], ll.entry_c, 0x7604u));
                        const uint32_t m0 = lds32(prmt(w[t], ll.mask_c, 0x7614u));
                        const uint2 e1 = lds64(prmt(w[t], ll.entry_c, 0x7624u));
                        const uint32_t m1 = lds32(prmt(w[t], ll.mask_c, 0x7634u));
                        uint32_t m0s, m1s;
                        asm("mad.lo.u32 %0, %1, 2, 0;" : "=r"(m0s) : "r"(m0));
                        asm("mad.lo.u32 %0, %1, 2, 0;" : "=r"(m1s) : "r"(m1));
                        d0 = make_uint2(e0.x ^ (m0 & 0x22222222u), e0.y ^ (m0s & 0x22222222u));
                        d1 = make_uint2(e1.x ^ (m1 & 0x22222222u), e1.y ^ (m1s & 0x22222222u));
                    } else {
                        d0 = decode8_fp6<0>(w[t], ll);
                        d1 = decode8_fp6<1>(w[t], ll);
                    }
                    r0[8 * i + 2 * t] = d0.x; r0[8 * i + 2 * t + 1] = d0.y;
                    r1[8 * i + 2 * t] = d1.x; r1[8 * i + 2 * t + 1] = d1.y;
                }
            }
            if (VAR & 2) {
#pragma unroll
                for (int i = 0; i < 16; ++i) sink ^= r0[i] ^ r1[i];
            } else {
                tmem_st16(colbase + g2 * 8, r0);
                tmem_st16(colbase + 32 + g2 * 8, r1);
            }
        }
        if (!(VAR & 2)) tmem_wait_st();
        if (VAR & 8) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars[q & 7]));
            if (!mbar_try_wait(smem_u32(&bars[q & 7]), (it + 1) & 1)) sink += 1;
            tc_fence_after();
        }
    }
    const long long t1 = clock64();
    __syncthreads();
    if (tid == 0) cyc[blockIdx.x] = t1 - t0;
    out[blockIdx.x * blockDim.x + tid] = sink;
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, 512);
    (void)nwarps;
}

template <int VAR, int G>
void run(const char *name, uint32_t *out, long long *cyc) {
    const int smem = 2048 + 65536 + 65536 + 32768;
    cudaFuncSetAttribute(k<VAR, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    for (int warps : {16, 20, 24, 32}) {
        const int iters = 2000;
        k<VAR, G><<<148, warps * 32, smem>>>(out, iters, cyc);
        cudaError_t e = cudaDeviceSynchronize();
        double c = 0;
        for (int i = 0; i < 148; ++i) c += cyc[i];
        c /= 148;
        const double tiles = (double)(warps / 4) * iters * G;
        printf("%-44s G=%d warps=%2d: %.1f cycles per tile  (%s)\n", name, G, warps, c / tiles, cudaGetErrorString(e));
        if (e != cudaSuccess) exit(1);
    }
}

int main() {
    uint32_t *out;
    long long *cyc;
    cudaMalloc(&out, 148 * 1024 * 4);
    cudaMallocManaged(&cyc, 148 * 8);
    run<0, 2>("8-byte entry, shf, lds.128 codes, st+wait", out, cyc);
    run<1, 2>("8-byte entry, imad (the product's decode)", out, cyc);
    run<1, 4>("8-byte entry, imad, four k-tiles per step", out, cyc);
    run<3, 2>("8-byte entry, imad, NO tcgen05.st", out, cyc);
    run<5, 2>("8-byte entry, imad, codes via tcgen05.ld", out, cyc);
    run<9, 2>("8-byte entry, imad, st+wait+arrive+fences", out, cyc);
    run<17, 2>("4-byte nibble entry, imad, st+wait", out, cyc);
    run<19, 2>("4-byte nibble entry, imad, NO tcgen05.st", out, cyc);
    return 0;
}
