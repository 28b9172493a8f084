// Decode-only kernel: tiled codes -> logical [N, K] weights, through the same table and
// XOR decode core that the matmul kernels use, so a bit-exact check of its output is a
// check of the decode stage itself.
#pragma once
#include "dmm_common.cuh"
#include "dmm_launch.h"

namespace dmm {

constexpr int kDecodeThreads = 512;

// Re-tiles codes from the layout of fast_decode_matmul_cuda -- flat uint32 [N/32][K/16][lane:32],
// word = code(n = 32*nb + lane, j = 2*kp) | code(j = 2*kp + 1) << 16, the completion this build
// defines for the reference's lane-per-column reads (fast_decode_matmul_cuda.cu:106,110-113,130) --
// into the tile layout [N/16][K/32][g:8][t:4][h:2] that every kernel of this library streams.
// One warp per (32-row block, k-tile): 256 contiguous bytes in, 256 contiguous bytes out; lane l
// holds the four codes of row 32*nb + l and trades two of them with lane l ^ 8 (rows g and g + 8
// of a strip share a 32-bit word of the tile layout).
__global__ void __launch_bounds__(256) retile_fast_kernel(const uint32_t *__restrict__ fast, uint32_t *__restrict__ tiled,
                                                          long long N, long long K) {
    const long long KT = K / 32;
    const long long warp = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= (N / 32) * KT) return;
    const long long nb = warp / KT, kt = warp - nb * KT;
    const uint32_t *src = fast + (nb * (K / 16) + 2 * kt) * 32;
    const uint32_t w0 = __ldg(src + lane), w1 = __ldg(src + 32 + lane);  // codes j = 4kt, 4kt+1 | 4kt+2, 4kt+3
    const uint32_t p0 = __shfl_xor_sync(0xffffffffu, w0, 8), p1 = __shfl_xor_sync(0xffffffffu, w1, 8);
    const int strip = lane >> 4, h = (lane >> 3) & 1, g = lane & 7;
    // word (g, t) of the tile layout = code of row g (low half) | code of row g + 8 (high half)
    uint2 out;
    if (h == 0) {  // this lane is row g: writes t = 0, 1 from its w0 and the partner's w0
        out.x = (w0 & 0xFFFFu) | (p0 << 16);
        out.y = (w0 >> 16) | (p0 & 0xFFFF0000u);
    } else {       // this lane is row g + 8: writes t = 2, 3 from the partner's w1 and its own
        out.x = (p1 & 0xFFFFu) | (w1 << 16);
        out.y = (p1 >> 16) | (w1 & 0xFFFF0000u);
    }
    uint32_t *dst = tiled + ((2 * nb + strip) * KT + kt) * 32 + g * 4 + h * 2;
    *reinterpret_cast<uint2 *>(dst) = out;
}

inline int launch_retile_fast(const void *fast, void *tiled, long long N, long long K, cudaStream_t stream) {
    const long long warps = (N / 32) * (K / 32);
    const unsigned blocks = static_cast<unsigned>((warps + 7) / 8);
    retile_fast_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint32_t *>(fast),
                                                   reinterpret_cast<uint32_t *>(tiled), N, K);
    return cudaGetLastError();
}


// One thread per 32-bit word of the tile layout (two codes: strip rows g and g+8).
template <bool kF16>
__global__ void __launch_bounds__(kDecodeThreads) decode_kernel(const uint32_t *__restrict__ words,
                                                               const void *__restrict__ cb, int cb_is_f16,
                                                               void *__restrict__ w_out, long long N, long long K,
                                                               int sign_convention, unsigned dyn_smem_bytes) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t lut_addr = (base + 0xFFFFu) & ~0xFFFFu;
    if (lut_addr + kLutBytes > base + dyn_smem_bytes) {
        if (threadIdx.x == 0) raise_status(DMM_STATUS_BAD_SMEM);
        return;
    }
    const bool bad = lut_fill(lut_addr, cb, cb_is_f16, sign_convention, kF16 ? kFmtOffset : kFmtTwos, threadIdx.x,
                              kDecodeThreads);
    if (bad) raise_status(DMM_STATUS_BAD_CODEBOOK);
    __syncthreads();
    const LutLane ll = lut_lane(lut_addr, threadIdx.x & 31);

    const long long KT = K / 32;
    const long long total = N * K / 16;  // words
    for (long long wi = blockIdx.x * static_cast<long long>(kDecodeThreads) + threadIdx.x; wi < total;
         wi += static_cast<long long>(gridDim.x) * kDecodeThreads) {
        const long long strip = wi / (KT * 32);
        const long long rem = wi - strip * KT * 32;
        const long long kt = rem >> 5;
        const int l = static_cast<int>(rem & 31), g = l >> 2, t = l & 3;
        const uint32_t word = __ldg(words + wi);
        const uint2 d0 = decode8<0>(word, ll), d1 = decode8<1>(word, ll);
        const long long n0 = strip * 16 + g, k0 = 32 * kt + 8 * t;
        if constexpr (kF16) {
            uint32_t a[4], b[4];
            bytes_to_half2(d0, a);
            bytes_to_half2(d1, b);
            const __half2 quarter = __float2half2_rn(0.25f);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                __half2 ha = __hmul2(*reinterpret_cast<__half2 *>(&a[i]), quarter);
                __half2 hb = __hmul2(*reinterpret_cast<__half2 *>(&b[i]), quarter);
                a[i] = *reinterpret_cast<uint32_t *>(&ha);
                b[i] = *reinterpret_cast<uint32_t *>(&hb);
            }
            __half *w = reinterpret_cast<__half *>(w_out);
            *reinterpret_cast<uint4 *>(w + n0 * K + k0) = make_uint4(a[0], a[1], a[2], a[3]);
            *reinterpret_cast<uint4 *>(w + (n0 + 8) * K + k0) = make_uint4(b[0], b[1], b[2], b[3]);
        } else {
            int8_t *w = reinterpret_cast<int8_t *>(w_out);
            *reinterpret_cast<uint2 *>(w + n0 * K + k0) = d0;
            *reinterpret_cast<uint2 *>(w + (n0 + 8) * K + k0) = d1;
        }
    }
}

inline int launch_decode(const void *codes, const void *cb, int cb_is_f16, void *w_out, long long N, long long K,
                         int sign_convention, int num_sms, cudaStream_t stream) {
    constexpr unsigned kDyn = 0xFFFFu + kLutBytes + 1;
    const long long total = N * K / 16;
    long long blocks = (total + kDecodeThreads - 1) / kDecodeThreads;
    if (blocks > num_sms) blocks = num_sms;
    if (blocks < 1) blocks = 1;
    cudaError_t err;
    if (cb_is_f16) {
        err = cudaFuncSetAttribute(decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDyn);
        if (err != cudaSuccess) return err;
        decode_kernel<true><<<(unsigned)blocks, kDecodeThreads, kDyn, stream>>>(
            reinterpret_cast<const uint32_t *>(codes), cb, 1, w_out, N, K, sign_convention, kDyn);
    } else {
        err = cudaFuncSetAttribute(decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDyn);
        if (err != cudaSuccess) return err;
        decode_kernel<false><<<(unsigned)blocks, kDecodeThreads, kDyn, stream>>>(
            reinterpret_cast<const uint32_t *>(codes), cb, 0, w_out, N, K, sign_convention, kDyn);
    }
    return cudaGetLastError();
}

}  // namespace dmm
