// C ABI of libdmm (declared in include/dmm.h): argument validation, workspace and
// per-device state, path selection, kernel launches.  The whole library is this one
// translation unit; the kernel headers are included below.
#include <atomic>
#include <mutex>

#include "dmm_common.cuh"
#include "dmm_decode.cuh"
#include "dmm_launch.h"
#include "dmm_stream.cuh"
#include "dmm_umma.cuh"
#include "dmm_tc.cuh"

namespace dmm {

constexpr int kMaxDevices = 64;

struct DeviceState {
    int num_sms = 0;
    void *workspace = nullptr;  // library-owned default workspace
    size_t workspace_bytes = 0;
    void *retile = nullptr;     // library-owned buffer for codes re-tiled from the fast layout
    size_t retile_bytes = 0;
    unsigned *chain_sync = nullptr;  // arrival counters of dmm_f16_chain (zero between launches)
    unsigned *xrank_counter = nullptr;  // number of dmm_xrank_barrier calls executed on this device
};

static std::mutex g_mutex;
static DeviceState g_dev[kMaxDevices];
static std::atomic<uint64_t> g_launches{0};
// dmm_hint_next_weights: what the calling host thread said its next-but-one product will stream
struct NextHint {
    const void *codes = nullptr;
    long long N = 0, K = 0;
};
static thread_local NextHint t_next_hint;

static std::atomic<long long> g_xrank_wait_cycles{kWaitLimitCycles};  // dmm_set_wait_limit_ms

static int current_device_state(DeviceState **out) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceState &d = g_dev[dev];
    if (d.num_sms == 0) {
        err = cudaDeviceGetAttribute(&d.num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (err != cudaSuccess) return err;
    }
    *out = &d;
    return 0;
}

// Size of the library's own workspace on first use: tickets for N up to 2^24 (4 MiB), stream-K partials
// at batch 64 (up to 256 CTAs: 16 MiB) and the activation planes for K up to 2^17 (16 MiB).
constexpr size_t kDefaultWorkspace = size_t(40) << 20;

static size_t ticket_bytes(long long N) {
    const size_t b = static_cast<size_t>(N / 16) * sizeof(unsigned);
    return (b + 255) & ~static_cast<size_t>(255);
}

// Every path shares the ticket block; the partial block is sized for the widest path
// that a batch of M columns can take (tcgen05, fp16 operands); behind it sits the buffer of
// pre-split activation planes of the fp8-operand path (up to 32 padded rows x K x 4 planes).
static size_t partial_bytes(long long M, int num_sms) {
    size_t per_slot = kPartialValues;
    const size_t umma = static_cast<size_t>(umma_partial_values(M > 64 ? 64 : M, false));
    if (umma > per_slot) per_slot = umma;
    return static_cast<size_t>(num_sms) * 2 * per_slot * 4;
}
static size_t planes_offset(long long M, long long N, int num_sms) {
    return (ticket_bytes(N) + partial_bytes(M, num_sms) + 255) & ~static_cast<size_t>(255);
}
static size_t workspace_need(long long M, long long N, long long K, int num_sms) {
    return planes_offset(M, N, num_sms) + static_cast<size_t>(K) * 128;
}

// Returns the workspace to use: the caller's (checked for size) or the library's own,
// grown on demand.  The ticket counters must be zero before the first launch; the
// library's buffer is cleared when it is (re)allocated, a caller's buffer by the caller.
static int resolve_workspace(DeviceState *d, long long M, long long N, long long K, void *user, size_t user_bytes,
                             cudaStream_t stream, void **ws) {
    const size_t need = workspace_need(M, N, K, d->num_sms);
    if (user != nullptr) {
        if (user_bytes < need) return DMM_ERR_WORKSPACE;
        if (reinterpret_cast<uintptr_t>(user) % 256 != 0) return DMM_ERR_ALIGN;
        *ws = user;
        return 0;
    }
    std::lock_guard<std::mutex> lock(g_mutex);
    if (d->workspace_bytes < need) {
        // Allocation is not possible while the stream is being captured into a graph.
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        cudaError_t err = cudaStreamIsCapturing(stream, &cap);
        if (err != cudaSuccess) return err;
        if (cap != cudaStreamCaptureStatusNone) return DMM_ERR_WORKSPACE;
        // The first allocation covers every call up to batch 64 and K = 131072 (kDefaultWorkspace).
        // A later, larger need gets a new buffer; the old one is parked, never freed: kernels already
        // enqueued and CUDA graphs captured earlier keep using it.
        const size_t bytes = need < kDefaultWorkspace ? kDefaultWorkspace : need;
        void *fresh = nullptr;
        err = cudaMalloc(&fresh, bytes);
        if (err != cudaSuccess) return err;
        err = cudaMemsetAsync(fresh, 0, bytes, stream);  // the ticket counters start at zero
        if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
        if (err != cudaSuccess) return err;
        d->workspace = fresh;  // (an outgrown buffer stays allocated until the process exits)
        d->workspace_bytes = bytes;
    }
    *ws = d->workspace;
    return 0;
}

// Codes given in the fast layout are re-tiled into a library-owned buffer (grown on demand) and
// the call goes on with the tile layout: one extra pass over the codes.  The reference's fast
// kernel is an unbuilt prototype; this keeps its entry point usable, not fast.
static int retile_fast(DeviceState *d, const void *codes, long long N, long long K, cudaStream_t stream,
                       const void **tiled) {
    if (N % 32 != 0) return DMM_ERR_SHAPE;
    const size_t need = static_cast<size_t>(N) * static_cast<size_t>(K) / 4;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (d->retile_bytes < need) {
            // as for the workspace: no allocation under stream capture, and an outgrown buffer is parked,
            // never freed (work already enqueued and graphs captured earlier keep using it)
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            cudaError_t err = cudaStreamIsCapturing(stream, &cap);
            if (err != cudaSuccess) return err;
            if (cap != cudaStreamCaptureStatusNone) return DMM_ERR_WORKSPACE;
            void *fresh = nullptr;
            err = cudaMalloc(&fresh, need);
            if (err != cudaSuccess) return err;
            d->retile = fresh;
            d->retile_bytes = need;
        }
    }
    const int rc = launch_retile_fast(codes, d->retile, N, K, stream);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (rc) return rc;
    *tiled = d->retile;
    return 0;
}

static bool aligned16(const void *p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

static int check_common(const void *x, const void *codes, const void *cb, const void *out, long long M, long long N,
                        long long K, int sign_convention, int layout) {
    if (!x || !codes || !cb || !out) return DMM_ERR_NULL;
    if (M < 1 || N < 16 || K < 32 || N % 16 != 0 || K % 32 != 0) return DMM_ERR_SHAPE;
    if (M > (1ll << 20) || N > (1ll << 24) || K > (1ll << 17)) return DMM_ERR_SHAPE;
    if (sign_convention != DMM_SIGN_SLOW && sign_convention != DMM_SIGN_FAST) return DMM_ERR_ARG;
    if (layout != DMM_LAYOUT_TILE && layout != DMM_LAYOUT_FAST) return DMM_ERR_ARG;
    if (!aligned16(x) || !aligned16(codes) || !aligned16(cb) || !aligned16(out)) return DMM_ERR_ALIGN;
    return 0;
}

// Streams the weights once per chunk of 16 batch columns.
static int run_stream(int family, const void *x, const void *codes, const void *cb, int cb_is_f16, float scale,
                      void *out, long long M, long long N, long long K, int sign_convention, unsigned flags,
                      void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    DeviceState *d = nullptr;
    int rc = current_device_state(&d);
    if (rc) return rc;
    void *ws = nullptr;
    rc = resolve_workspace(d, M, N, K, workspace, workspace_bytes, stream, &ws);
    if (rc) return rc;
    const size_t x_elem = family == 0 ? 1 : 2;
    for (long long m0 = 0; m0 < M; m0 += 16) {
        StreamParams p = {};
        p.x = reinterpret_cast<const uint8_t *>(x) + static_cast<size_t>(m0) * K * x_elem;
        p.codes = codes;
        p.cb = cb;
        p.out = reinterpret_cast<uint8_t *>(out) + static_cast<size_t>(m0) * N * 4;
        p.tickets = reinterpret_cast<unsigned *>(ws);
        p.partials = reinterpret_cast<uint8_t *>(ws) + ticket_bytes(N);
        p.M = M - m0 < 16 ? M - m0 : 16;
        p.N = N;
        p.K = K;
        p.scale = scale;
        p.accumulate = (flags & DMM_FLAG_ACCUMULATE) ? 1 : 0;
        p.sign_convention = sign_convention;
        p.cb_is_f16 = cb_is_f16;
        rc = launch_stream(family, p, d->num_sms, (flags & DMM_FLAG_PDL) != 0, stream);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if (rc) return rc;
    }
    return 0;
}


// tcgen05 path: one launch per chunk of 64 batch columns (32 for the fp6/fp8 operand policy,
// preceded by planes_kernel when the chunk has at least kPlanesMinBatch rows).
// Tensor-parallel extras of one call (dmm_f16_fused_tp).
struct TpArgs {
    float *const *peer_out = nullptr;
    int n_peers = 0;
    float *move_src = nullptr, *move_dst = nullptr;
    long long move_count = 0;
    // slots form (dmm_f16_tp_produce / dmm_f16_tp_consume)
    int mode = 0, rank = 0, world = 0;
    unsigned *const *flags = nullptr;
    long long count = 0;
    float *h_out = nullptr;
};

static int run_umma(bool f8, const void *x, int x_kind, long long x_ld, long long x_gap, const void *codes,
                    const void *cb16, float scale, float *out, long long M, long long N, long long K,
                    int sign_convention, unsigned flags, void *workspace, size_t workspace_bytes, cudaStream_t stream,
                    float *zero_ptr = nullptr, long long zero_count = 0, const TpArgs *tp = nullptr, bool fast_layout = false) {
    DeviceState *d = nullptr;
    int rc = current_device_state(&d);
    if (rc) return rc;
    void *ws = nullptr;
    rc = resolve_workspace(d, M, N, K, workspace, workspace_bytes, stream, &ws);
    if (rc) return rc;
    const long long step = f8 ? 32 : 64;
    const bool pdl = (flags & DMM_FLAG_PDL) != 0;
    for (long long m0 = 0; m0 < M; m0 += step) {
        UmmaParams p = {};
        p.x = reinterpret_cast<const uint8_t *>(x) + static_cast<size_t>(m0) * x_ld * (x_kind == DMM_X_F16 ? 2 : 4);
        p.M = M - m0 < step ? M - m0 : step;
        if (f8 && p.M >= kPlanesMinBatch && !(tp != nullptr && tp->mode == 3)) {
            // split the activations into E5M2 planes once, instead of once per CTA inside the kernel
            uint8_t *planes = reinterpret_cast<uint8_t *>(ws) + planes_offset(M, N, d->num_sms);
            rc = launch_planes(p.x, x_kind, x_ld, x_gap, static_cast<int>(p.M), K, planes, pdl, stream);
            g_launches.fetch_add(1, std::memory_order_relaxed);
            if (rc) return rc;
            p.x_planes = planes;
        }
        p.x_mode = x_kind;
        p.x_ld = x_ld;
        p.x_gap = x_gap;
        p.codes = codes;
        p.cb = cb16;
        p.out = out + static_cast<size_t>(m0) * N;
        p.tickets = reinterpret_cast<unsigned *>(ws);
        p.partials = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(ws) + ticket_bytes(N));
        p.N = N;
        p.K = K;
        // accumulators hold sum(x * q / 8) (fp6 weights) or sum(x * q) (fp16 weights); weight = q / 4
        p.scale = f8 ? 2.0f * scale : 0.25f * scale;
        p.accumulate = (flags & DMM_FLAG_ACCUMULATE) ? 1 : 0;
        p.atomic_reduce = (flags & DMM_FLAG_ATOMIC) ? 1 : 0;
        p.sign_convention = sign_convention;
        p.fast_layout = fast_layout ? 1 : 0;
        if (m0 == 0) {
            p.zero_ptr = zero_ptr;
            p.zero_count = zero_count;
            if (tp != nullptr) {
                p.move_src = tp->move_src;
                p.move_dst = tp->move_dst;
                p.move_count = tp->move_count;
            }
        }
        if (tp != nullptr && tp->mode == 0) {
            p.n_peers = tp->n_peers;
            for (int r = 0; r < tp->n_peers; ++r) p.peer_out[r] = tp->peer_out[r] + static_cast<size_t>(m0) * N;
        }
        if (tp != nullptr && tp->mode != 0) {
            p.tp_mode = tp->mode;
            p.tp_rank = tp->rank;
            p.tp_world = tp->world;
            p.tp_count = tp->count;
            p.tp_wait = g_xrank_wait_cycles.load(std::memory_order_relaxed);
            p.h_out = tp->h_out;
            for (int r = 0; r < tp->world; ++r) {
                p.peer_out[r] = tp->peer_out[r];
                p.tp_flags[r] = tp->flags[r];
            }
        }
        if (m0 + step >= M && t_next_hint.codes != nullptr) {  // the last launch of this call prefetches for the next call
            p.next_codes = t_next_hint.codes;
            p.next_N = t_next_hint.N;
            p.next_K = t_next_hint.K;
            t_next_hint = NextHint();
        }
        // 17 to 32 batch rows (128 MMA columns) run on the kernel of dmm_tc.cuh, measured faster there;
        // everything else on the kernel of dmm_umma.cuh
        rc = (f8 && p.M > 16 && !fast_layout) ? launch_tc_wide(p, d->num_sms, pdl, stream) : launch_umma(f8, p, d->num_sms, pdl, stream);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if (rc) return rc;
    }
    return 0;
}

// Integer family on the tcgen05 kernel: one launch per chunk of 32 batch rows.
static int run_umma_i8(const void *x, const void *codes, const void *cb64, int32_t *out, long long M, long long N,
                       long long K, int sign_convention, unsigned flags, void *workspace, size_t workspace_bytes,
                       cudaStream_t stream, bool fast_layout) {
    DeviceState *d = nullptr;
    int rc = current_device_state(&d);
    if (rc) return rc;
    void *ws = nullptr;
    rc = resolve_workspace(d, M, N, K, workspace, workspace_bytes, stream, &ws);
    if (rc) return rc;
    // Integer sums do not depend on their order, so partial super-tiles are always added with
    // atomics (no workspace round trip, no ticket); a plain product clears the output first.
    if (!(flags & DMM_FLAG_ACCUMULATE)) {
        const cudaError_t err = cudaMemsetAsync(out, 0, static_cast<size_t>(M) * static_cast<size_t>(N) * sizeof(int32_t), stream);
        if (err != cudaSuccess) return err;
    }
    for (long long m0 = 0; m0 < M; m0 += 32) {
        UmmaParams p = {};
        p.x = reinterpret_cast<const int8_t *>(x) + static_cast<size_t>(m0) * K;
        p.x_ld = K;
        p.codes = codes;
        p.cb = cb64;
        p.out = reinterpret_cast<float *>(out + static_cast<size_t>(m0) * N);  // int32 behind the kernel's generic pointer
        p.tickets = reinterpret_cast<unsigned *>(ws);
        p.partials = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(ws) + ticket_bytes(N));
        p.M = M - m0 < 32 ? M - m0 : 32;
        p.N = N;
        p.K = K;
        p.scale = 1.0f;
        p.accumulate = 1;
        p.atomic_reduce = 1;
        p.sign_convention = sign_convention;
        p.fast_layout = fast_layout ? 1 : 0;
        rc = launch_umma_i8(p, d->num_sms, (flags & DMM_FLAG_PDL) != 0, stream);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if (rc) return rc;
    }
    return 0;
}

// ---------------------------------------------------------------------------------------
// Fixed scratch for dmm_f16_noalloc: ticket counters, then stream-K partials for up to
// kNoAllocMaxCtas CTAs of the fp8-operand tcgen05 kernel (2 slots x 2048 floats each).
// A file-scope device array: every GPU that loads the library carries it until exit.
// ---------------------------------------------------------------------------------------
constexpr int kNoAllocMaxCtas = 160;
constexpr long long kNoAllocMaxM = 8;
constexpr long long kNoAllocMaxN = 262144;  // 1024 super-tiles -> 4 KiB of tickets
constexpr size_t kNoAllocTicketBytes = 4096;
constexpr size_t kNoAllocBytes = kNoAllocTicketBytes + static_cast<size_t>(kNoAllocMaxCtas) * 2 * 2048 * sizeof(float);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];
static void *g_noalloc_ptr[kMaxDevices];  // device address of the array, per device, set on first use

// Device address of g_noalloc_scratch on the current device.  In host code the array's name
// is only a handle; the address a kernel can use comes from cudaGetSymbolAddress, asked once
// per device with that device current.
static int noalloc_scratch(void **out) {
    int dev = 0;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess) return err;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
        void *ptr = nullptr;
        err = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (err != cudaSuccess) return err;
        g_noalloc_ptr[dev] = ptr;
    }
    *out = g_noalloc_ptr[dev];
    return 0;
}

}  // namespace dmm

using namespace dmm;

extern "C" {

int dmm_i8(const int8_t *x, const int16_t *codes, const int64_t *cb64, int32_t *out, int64_t M, int64_t N, int64_t K,
           int sign_convention, int layout, unsigned flags, void *workspace, size_t workspace_bytes, void *stream) {
    int rc = check_common(x, codes, cb64, out, M, N, K, sign_convention, layout);
    if (rc) return rc;
    // the tcgen05 kernel streams either layout as it lies in memory
    if (layout == DMM_LAYOUT_FAST && N % 32 != 0) return DMM_ERR_SHAPE;
    return run_umma_i8(x, codes, cb64, out, M, N, K, sign_convention, flags, workspace, workspace_bytes,
                       static_cast<cudaStream_t>(stream), layout == DMM_LAYOUT_FAST);
}

int dmm_f16_fused(const void *x, int x_kind, int64_t x_ld, int64_t x_gap, const int16_t *codes, const void *cb16,
                  float scale, float *out, int64_t M, int64_t N, int64_t K, int sign_convention, int layout, int path,
                  unsigned flags, float *zero_ptr, int64_t zero_count, void *workspace, size_t workspace_bytes,
                  void *stream) {
    int rc = check_common(x, codes, cb16, out, M, N, K, sign_convention, layout);
    if (rc) return rc;
    if (path != DMM_PATH_AUTO && path != DMM_PATH_GEMV && path != DMM_PATH_TCGEN05 && path != DMM_PATH_TCGEN05_F8)
        return DMM_ERR_ARG;
    if (x_kind != DMM_X_F16 && x_kind != DMM_X_F32 && x_kind != DMM_X_F32_SILU_MUL) return DMM_ERR_ARG;
    if (x_ld < K || x_ld % 8 != 0 || x_gap % 4 != 0 || (x_kind == DMM_X_F32_SILU_MUL && x_gap + K > x_ld))
        return DMM_ERR_SHAPE;
    if (zero_count < 0 || (zero_count > 0 && zero_ptr == nullptr)) return DMM_ERR_ARG;
    if (path == DMM_PATH_AUTO) path = x_kind == DMM_X_F16 ? dmm_select_path(M, N, K) : DMM_PATH_TCGEN05_F8;
    bool fast_native = false;
    if (layout == DMM_LAYOUT_FAST) {
        if (N % 32 != 0) return DMM_ERR_SHAPE;
        if (path == DMM_PATH_TCGEN05_F8) {
            fast_native = true;  // streamed as it lies in memory
        } else {                 // the cross-check paths read the tile layout: re-tile first (one extra pass)
            DeviceState *d = nullptr;
            rc = current_device_state(&d);
            if (rc) return rc;
            const void *tiled = nullptr;
            rc = retile_fast(d, codes, N, K, static_cast<cudaStream_t>(stream), &tiled);
            if (rc) return rc;
            codes = reinterpret_cast<const int16_t *>(tiled);
        }
    }
    if (zero_count > 0 && path != DMM_PATH_TCGEN05 && path != DMM_PATH_TCGEN05_F8) return DMM_ERR_UNSUPPORTED;
    // fp32 inputs are converted by the loaders of the fp8-operand kernel only
    if (x_kind != DMM_X_F16 && path != DMM_PATH_TCGEN05_F8) return DMM_ERR_UNSUPPORTED;
    if (path == DMM_PATH_TCGEN05 || path == DMM_PATH_TCGEN05_F8)
        return run_umma(path == DMM_PATH_TCGEN05_F8, x, x_kind, x_ld, x_gap, codes, cb16, scale, out, M, N, K,
                        sign_convention, flags, workspace, workspace_bytes, static_cast<cudaStream_t>(stream), zero_ptr,
                        zero_count, nullptr, fast_native);
    if (x_ld != K) return DMM_ERR_UNSUPPORTED;
    // the streaming kernel accumulates quarter units: fold the 1/4 into the scale
    return run_stream(1, x, codes, cb16, 1, 0.25f * scale, out, M, N, K, sign_convention, flags, workspace,
                      workspace_bytes, static_cast<cudaStream_t>(stream));
}

int dmm_f16(const void *x, const int16_t *codes, const void *cb16, float scale, float *out, int64_t M, int64_t N,
            int64_t K, int sign_convention, int layout, int path, unsigned flags, void *workspace,
            size_t workspace_bytes, void *stream) {
    return dmm_f16_fused(x, DMM_X_F16, K, 0, codes, cb16, scale, out, M, N, K, sign_convention, layout, path, flags,
                         nullptr, 0, workspace, workspace_bytes, stream);
}

int dmm_f16_fused_tp(const void *x, int x_kind, int64_t x_ld, int64_t x_gap, const int16_t *codes, const void *cb16,
                     float scale, float *const *peer_out, int n_peers, int64_t M, int64_t N, int64_t K,
                     int sign_convention, unsigned flags, float *zero_ptr, int64_t zero_count, float *move_src,
                     float *move_dst, int64_t move_count, void *stream) {
    if (!peer_out) return DMM_ERR_NULL;
    if (n_peers < 1 || n_peers > 8) return DMM_ERR_ARG;
    for (int r = 0; r < n_peers; ++r)
        if (!peer_out[r] || !aligned16(peer_out[r])) return peer_out[r] ? DMM_ERR_ALIGN : DMM_ERR_NULL;
    int rc = check_common(x, codes, cb16, peer_out[0], M, N, K, sign_convention, DMM_LAYOUT_TILE);
    if (rc) return rc;
    if (x_kind != DMM_X_F16 && x_kind != DMM_X_F32 && x_kind != DMM_X_F32_SILU_MUL) return DMM_ERR_ARG;
    if (x_ld < K || x_ld % 8 != 0 || x_gap % 4 != 0 || (x_kind == DMM_X_F32_SILU_MUL && x_gap + K > x_ld))
        return DMM_ERR_SHAPE;
    if (flags & ~DMM_FLAG_PDL) return DMM_ERR_ARG;
    if (zero_count < 0 || (zero_count > 0 && zero_ptr == nullptr)) return DMM_ERR_ARG;
    if (move_count < 0 || (move_count > 0 && (move_src == nullptr || move_dst == nullptr))) return DMM_ERR_ARG;
    TpArgs tp;
    tp.peer_out = peer_out;
    tp.n_peers = n_peers;
    tp.move_src = move_src;
    tp.move_dst = move_dst;
    tp.move_count = move_count;
    return run_umma(true, x, x_kind, x_ld, x_gap, codes, cb16, scale, peer_out[0], M, N, K, sign_convention,
                    flags | DMM_FLAG_ATOMIC | DMM_FLAG_ACCUMULATE, nullptr, 0, static_cast<cudaStream_t>(stream), zero_ptr,
                    zero_count, &tp);
}

static int check_tp_group(float *const *peer_slots, unsigned *const *peer_flags, int rank, int world) {
    if (!peer_slots || !peer_flags) return DMM_ERR_NULL;
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return DMM_ERR_ARG;
    for (int r = 0; r < world; ++r) {
        if (!peer_slots[r] || !peer_flags[r]) return DMM_ERR_NULL;
        if (!aligned16(peer_slots[r]) || !aligned16(peer_flags[r])) return DMM_ERR_ALIGN;
    }
    return 0;
}

int dmm_f16_tp_produce(const void *x, int x_kind, int64_t x_ld, int64_t x_gap, const int16_t *codes, const void *cb16,
                       float scale, float *const *peer_slots, unsigned *const *peer_flags, int rank, int world, int64_t M,
                       int64_t N, int64_t K, int sign_convention, unsigned flags, void *stream) {
    int rc = check_tp_group(peer_slots, peer_flags, rank, world);
    if (rc) return rc;
    rc = check_common(x, codes, cb16, peer_slots[rank], M, N, K, sign_convention, DMM_LAYOUT_TILE);
    if (rc) return rc;
    if (M > 8) return DMM_ERR_LIMIT;
    if (x_kind != DMM_X_F16 && x_kind != DMM_X_F32 && x_kind != DMM_X_F32_SILU_MUL) return DMM_ERR_ARG;
    if (x_ld < K || x_ld % 8 != 0 || x_gap % 4 != 0 || (x_kind == DMM_X_F32_SILU_MUL && x_gap + K > x_ld))
        return DMM_ERR_SHAPE;
    if (flags & ~DMM_FLAG_PDL) return DMM_ERR_ARG;
    TpArgs tp;
    tp.mode = 2;
    tp.rank = rank;
    tp.world = world;
    tp.peer_out = peer_slots;
    tp.flags = peer_flags;
    tp.count = M * N;
    return run_umma(true, x, x_kind, x_ld, x_gap, codes, cb16, scale, peer_slots[rank], M, N, K, sign_convention,
                    flags | DMM_FLAG_ATOMIC | DMM_FLAG_ACCUMULATE, nullptr, 0, static_cast<cudaStream_t>(stream), nullptr, 0, &tp);
}

int dmm_f16_tp_consume(const float *h_in, float *h_out, int64_t x_ld, const float *slots, const unsigned *flags_local,
                       int world, int64_t slot_count, const int16_t *codes, const void *cb16, float scale, float *out,
                       int64_t M, int64_t N, int64_t K, int sign_convention, unsigned flags, float *zero_ptr,
                       int64_t zero_count, void *stream) {
    if (!h_in || !h_out || !slots || !flags_local) return DMM_ERR_NULL;
    if (world < 1 || world > 8) return DMM_ERR_ARG;
    int rc = check_common(h_in, codes, cb16, out, M, N, K, sign_convention, DMM_LAYOUT_TILE);
    if (rc) return rc;
    if (M > 8) return DMM_ERR_LIMIT;
    if (!aligned16(h_out) || !aligned16(slots) || !aligned16(flags_local)) return DMM_ERR_ALIGN;
    if (x_ld != K || slot_count != M * K) return DMM_ERR_SHAPE;  // the residual stream is [M, K], a slot one copy of it
    if (zero_count < 0 || (zero_count > 0 && zero_ptr == nullptr)) return DMM_ERR_ARG;
    // the kernel finds "this rank's" slot array and flag words in entry `rank` of the per-rank tables:
    // a consumer only ever touches its own, so every entry names them and the rank is 0
    float *slot_tab[8];
    unsigned *flag_tab[8];
    for (int r = 0; r < 8; ++r) {
        slot_tab[r] = const_cast<float *>(slots);
        flag_tab[r] = const_cast<unsigned *>(flags_local);
    }
    TpArgs tp;
    tp.mode = 3;
    tp.rank = 0;
    tp.world = world;
    tp.peer_out = slot_tab;
    tp.flags = flag_tab;
    tp.count = slot_count;
    tp.h_out = h_out;
    return run_umma(true, h_in, DMM_X_F32, x_ld, 0, codes, cb16, scale, out, M, N, K, sign_convention,
                    flags | DMM_FLAG_ATOMIC | DMM_FLAG_ACCUMULATE, nullptr, 0, static_cast<cudaStream_t>(stream), zero_ptr,
                    zero_count, &tp);
}

int dmm_tp_finalize(const float *h_in, float *h_out, const float *slots, const unsigned *flags_local, int world,
                    int64_t count, void *stream) {
    if (!h_in || !h_out || !slots || !flags_local) return DMM_ERR_NULL;
    if (world < 1 || world > 8) return DMM_ERR_ARG;
    if (count < 4 || count % 4 != 0) return DMM_ERR_SHAPE;
    if (!aligned16(h_in) || !aligned16(h_out) || !aligned16(slots)) return DMM_ERR_ALIGN;
    TpFinalizeParams fp = {};
    fp.h_in = h_in;
    fp.h_out = h_out;
    fp.slots = slots;
    fp.flags = flags_local;
    fp.count = count;
    fp.world = world;
    fp.wait_limit = g_xrank_wait_cycles.load(std::memory_order_relaxed);
    long long blocks = (count / 4 + 255) / 256;
    if (blocks > 16) blocks = 16;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(256);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaLaunchKernelEx(&cfg, tp_finalize_kernel, fp);
}

int dmm_xrank_barrier(unsigned *const *peer_flags, int rank, int world, void *stream) {
    if (!peer_flags) return DMM_ERR_NULL;
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return DMM_ERR_ARG;
    DeviceState *d = nullptr;
    int rc = current_device_state(&d);
    if (rc) return rc;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (d->xrank_counter == nullptr) {
            cudaError_t err = cudaMalloc(reinterpret_cast<void **>(&d->xrank_counter), 256);
            if (err != cudaSuccess) return err;
            err = cudaMemset(d->xrank_counter, 0, 256);
            if (err != cudaSuccess) return err;
        }
    }
    XrankBarrierParams bp = {};
    for (int r = 0; r < world; ++r) {
        if (!peer_flags[r]) return DMM_ERR_NULL;
        bp.flags[r] = peer_flags[r];
    }
    bp.counter = d->xrank_counter;
    bp.rank = rank;
    bp.world = world;
    bp.wait_limit = g_xrank_wait_cycles.load(std::memory_order_relaxed);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaLaunchKernelEx(&cfg, xrank_barrier_kernel, bp);
}

int dmm_xrank_allreduce_add(float *dst, const float *const *peer_src, float *zero_local, int64_t count,
                            unsigned *const *peer_flags, int rank, int world, void *stream) {
    if (!dst || !peer_src || !peer_flags) return DMM_ERR_NULL;
    if (world < 1 || world > 8 || rank < 0 || rank >= world) return DMM_ERR_ARG;
    if (count < 4 || count % 4 != 0) return DMM_ERR_SHAPE;
    if (!aligned16(dst) || (zero_local && !aligned16(zero_local))) return DMM_ERR_ALIGN;
    DeviceState *d = nullptr;
    int rc = current_device_state(&d);
    if (rc) return rc;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (d->xrank_counter == nullptr) {
            cudaError_t err = cudaMalloc(reinterpret_cast<void **>(&d->xrank_counter), 256);
            if (err != cudaSuccess) return err;
            err = cudaMemset(d->xrank_counter, 0, 256);
            if (err != cudaSuccess) return err;
        }
    }
    XrankAllreduceParams ap = {};
    for (int r = 0; r < world; ++r) {
        if (!peer_src[r] || !peer_flags[r]) return DMM_ERR_NULL;
        if (!aligned16(peer_src[r])) return DMM_ERR_ALIGN;
        ap.peer_src[r] = peer_src[r];
        ap.flags[r] = peer_flags[r];
    }
    ap.counter = d->xrank_counter;       // word 0: barriers / all-reduces done; word 16: block ticket
    ap.ticket = d->xrank_counter + 16;
    ap.dst = dst;
    ap.zero_local = zero_local;
    ap.count = count;
    ap.rank = rank;
    ap.world = world;
    ap.wait_limit = g_xrank_wait_cycles.load(std::memory_order_relaxed);
    long long blocks = (count / 4 + 255) / 256;
    if (blocks > 16) blocks = 16;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(blocks));
    cfg.blockDim = dim3(256);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cudaLaunchKernelEx(&cfg, xrank_allreduce_kernel, ap);
}

int dmm_f16_chain(const dmm_chain_op *ops, int n_ops, const void *cb16, int64_t M, int sign_convention,
                  unsigned flags, void *stream) {
    if (!ops || !cb16) return DMM_ERR_NULL;
    if (n_ops < 2 || n_ops > DMM_CHAIN_MAX_OPS) return DMM_ERR_ARG;
    if (M < 1 || M > 8) return DMM_ERR_LIMIT;
    if (flags & ~DMM_FLAG_PDL) return DMM_ERR_ARG;
    DeviceState *d = nullptr;
    int rc = current_device_state(&d);
    if (rc) return rc;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        if (d->chain_sync == nullptr) {
            cudaError_t err = cudaMalloc(reinterpret_cast<void **>(&d->chain_sync), 256);
            if (err != cudaSuccess) return err;
            err = cudaMemset(d->chain_sync, 0, 256);
            if (err != cudaSuccess) return err;
        }
    }
    UmmaParams p[DMM_CHAIN_MAX_OPS] = {};
    for (int i = 0; i < n_ops; ++i) {
        const dmm_chain_op &o = ops[i];
        rc = check_common(o.x, o.codes, cb16, o.out, M, o.N, o.K, sign_convention, DMM_LAYOUT_TILE);
        if (rc) return rc;
        if (o.x_kind != DMM_X_F16 && o.x_kind != DMM_X_F32 && o.x_kind != DMM_X_F32_SILU_MUL) return DMM_ERR_ARG;
        if (o.x_ld < o.K || o.x_ld % 8 != 0 || o.x_gap % 4 != 0 || (o.x_kind == DMM_X_F32_SILU_MUL && o.x_gap + o.K > o.x_ld))
            return DMM_ERR_SHAPE;
        if (o.zero_count < 0 || (o.zero_count > 0 && o.zero_ptr == nullptr)) return DMM_ERR_ARG;
        p[i].x = o.x;
        p[i].x_mode = o.x_kind;
        p[i].x_ld = o.x_ld;
        p[i].x_gap = o.x_gap;
        p[i].codes = o.codes;
        p[i].cb = cb16;
        p[i].out = o.out;
        p[i].M = M;
        p[i].N = o.N;
        p[i].K = o.K;
        p[i].scale = 2.0f * o.scale;  // accumulators hold sum(x * q / 8), weight = q / 4
        p[i].accumulate = 1;
        p[i].atomic_reduce = 1;
        p[i].sign_convention = sign_convention;
        p[i].zero_ptr = o.zero_ptr;
        p[i].zero_count = o.zero_count;
    }
    rc = launch_umma_chain(p, n_ops, d->chain_sync, d->num_sms, (flags & DMM_FLAG_PDL) != 0,
                           static_cast<cudaStream_t>(stream));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return rc;
}

int dmm_f16_noalloc(const void *x, const int16_t *codes, const void *cb16, float scale, float *out, int64_t M,
                    int64_t N, int64_t K, int sign_convention, unsigned flags, void *stream) {
    int rc = check_common(x, codes, cb16, out, M, N, K, sign_convention, DMM_LAYOUT_TILE);
    if (rc) return rc;
    if (M > kNoAllocMaxM || N > kNoAllocMaxN) return DMM_ERR_LIMIT;
    // the scratch holds stream-K partials only: the atomic epilogue has no use for it and is not offered here
    if (flags & ~(DMM_FLAG_ACCUMULATE | DMM_FLAG_PDL)) return DMM_ERR_ARG;
    DeviceState *d = nullptr;
    rc = current_device_state(&d);
    if (rc) return rc;
    void *ws = nullptr;
    rc = noalloc_scratch(&ws);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left.  Partials are always written before
    // they are read; the ticket counters must start at zero, so clear them (a call that was
    // cut short by a device-side timeout could have left some behind).
    cudaError_t err = cudaMemsetAsync(ws, 0, kNoAllocTicketBytes, st);
    if (err != cudaSuccess) return err;
    UmmaParams p = {};
    p.x = x;
    p.x_mode = DMM_X_F16;
    p.x_ld = K;
    p.codes = codes;
    p.cb = cb16;
    p.out = out;
    p.tickets = reinterpret_cast<unsigned *>(ws);
    p.partials = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(ws) + kNoAllocTicketBytes);
    p.M = M;
    p.N = N;
    p.K = K;
    p.scale = 2.0f * scale;
    p.accumulate = (flags & DMM_FLAG_ACCUMULATE) ? 1 : 0;
    p.sign_convention = sign_convention;
    const int ctas = d->num_sms < kNoAllocMaxCtas ? d->num_sms : kNoAllocMaxCtas;
    rc = launch_umma(true, p, ctas, (flags & DMM_FLAG_PDL) != 0, st);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return rc;
}

int dmm_decode(const int16_t *codes, const void *cb, int cb_is_f16, void *W_out, int64_t N, int64_t K,
               int sign_convention, int layout, void *stream) {
    if (!codes || !cb || !W_out) return DMM_ERR_NULL;
    if (N < 16 || K < 32 || N % 16 != 0 || K % 32 != 0) return DMM_ERR_SHAPE;
    if (sign_convention != DMM_SIGN_SLOW && sign_convention != DMM_SIGN_FAST) return DMM_ERR_ARG;
    if (layout != DMM_LAYOUT_TILE && layout != DMM_LAYOUT_FAST) return DMM_ERR_ARG;
    if (!aligned16(codes) || !aligned16(cb) || !aligned16(W_out)) return DMM_ERR_ALIGN;
    DeviceState *d = nullptr;
    int rc = current_device_state(&d);
    if (rc) return rc;
    if (layout == DMM_LAYOUT_FAST) {
        const void *tiled = nullptr;
        rc = retile_fast(d, codes, N, K, static_cast<cudaStream_t>(stream), &tiled);
        if (rc) return rc;
        codes = reinterpret_cast<const int16_t *>(tiled);
    }
    rc = launch_decode(codes, cb, cb_is_f16 ? 1 : 0, W_out, N, K, sign_convention, d->num_sms,
                       static_cast<cudaStream_t>(stream));
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return rc;
}

size_t dmm_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    (void)K;
    if (N < 16) return 0;
    DeviceState *d = nullptr;
    int sms = 256;
    if (current_device_state(&d) == 0 && d->num_sms > 0) sms = d->num_sms;
    return workspace_need(M, N, K, sms);
}

int dmm_status(unsigned *status_out) {
    if (!status_out) return DMM_ERR_NULL;
    cudaError_t err = cudaDeviceSynchronize();
    if (err != cudaSuccess) return err;
    unsigned v = 0;
    err = cudaMemcpyFromSymbol(&v, g_status, sizeof(v));
    if (err != cudaSuccess) return err;
    const unsigned zero = 0;
    err = cudaMemcpyToSymbol(g_status, &zero, sizeof(zero));
    if (err != cudaSuccess) return err;
    if (v != 0) {
        // a chain that gave up may have left its arrival counters behind
        DeviceState *d = nullptr;
        if (current_device_state(&d) == 0 && d->chain_sync != nullptr) {
            err = cudaMemset(d->chain_sync, 0, 256);
            if (err != cudaSuccess) return err;
        }
    }
    *status_out = v;
    return 0;
}

int dmm_select_path(int64_t M, int64_t N, int64_t K) {
    // Measured on B200: the fp6/fp8-operand kernel (32 batch rows per pass, planes split once by
    // planes_kernel from 4 rows on) beats the fp16-operand one at every batch size.
    (void)M;
    (void)N;
    (void)K;
    return DMM_PATH_TCGEN05_F8;
}

int dmm_set_wait_limit_ms(unsigned ms) {
    // about 2 clock cycles per nanosecond; 0 restores the default (about a quarter of a second)
    g_xrank_wait_cycles.store(ms == 0 ? kWaitLimitCycles : static_cast<long long>(ms) * 2000000ll, std::memory_order_relaxed);
    return 0;
}

int dmm_hint_next_weights(const int16_t *codes, int64_t N, int64_t K) {
    if (codes != nullptr && (N < 16 || K < 32 || N % 16 != 0 || K % 32 != 0 || !aligned16(codes))) return DMM_ERR_SHAPE;
    t_next_hint.codes = codes;
    t_next_hint.N = N;
    t_next_hint.K = K;
    return 0;
}

uint64_t dmm_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

const char *dmm_error_string(int code) {
    switch (code) {
        case DMM_OK: return "ok";
        case DMM_ERR_NULL: return "a required pointer is NULL";
        case DMM_ERR_SHAPE: return "bad shape: need M >= 1, N % 16 == 0, K % 32 == 0";
        case DMM_ERR_ALIGN: return "a pointer is not 16-byte aligned";
        case DMM_ERR_ARG: return "unknown enum value";
        case DMM_ERR_WORKSPACE: return "workspace too small (see dmm_workspace_bytes)";
        case DMM_ERR_UNSUPPORTED: return "shape or layout not implemented by the chosen path";
        case DMM_ERR_LIMIT: return "size beyond the fixed scratch of dmm_f16_noalloc (M <= 8, N <= 262144)";
        default: break;
    }
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown error";
}

const char *dmm_version(void) { return "0.1"; }


}  // extern "C"
