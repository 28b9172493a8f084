/*
 * dmm.h -- C ABI of libdmm, the B200 (sm_100a) codebook decode-and-matmul library.
 *
 * Every entry point takes plain device pointers and sizes, enqueues its work on the
 * given CUDA stream and returns immediately: it never synchronises the device, never
 * throws and never exits the process.  Return value: 0 = enqueued, negative = argument
 * error (DMM_ERR_*), positive = the cudaError_t of a failed runtime call.
 *
 * Data formats (shared by all entry points)
 *   code word      uint16: bits 0..7 codebook index, bits 8..14 seven stored sign bits,
 *                  bit 15 shift bit; the eighth sign is the parity of the seven.
 *   codes_tiled    int16, N*K/8 values in the tile layout of the reference's
 *                  transpose_tile() (test_decode_matmul.py:101-109):
 *                  [N/16][K/32][g:8][t:4][h:2], row n = 16*nt + 8*h + g, column j = 4*kt + t.
 *   codes_fast     the layout of fast_decode_matmul_cuda (DMM_LAYOUT_FAST): flat uint32
 *                  [N/32][K/16][lane:32], word = code(n = 32*nb + lane, j = 2*kp) |
 *                  code(j = 2*kp + 1) << 16 -- one word per lane, a warp covering 32 consecutive
 *                  output columns, as the reference's fast kernel reads them
 *                  (fast_decode_matmul_cuda.cu:106,110-113,130); that kernel's k addressing is
 *                  not self-consistent, so the k order is this library's completion of it.
 *                  Needs N % 32 == 0.  dmm_i8, dmm_f16 and dmm_f16_fused stream it as it lies in
 *                  memory on their default paths (own tensor map and lane-to-row mapping, no
 *                  extra pass).  Only the cross-check paths (DMM_PATH_GEMV, DMM_PATH_TCGEN05)
 *                  re-tile it into a library-owned device buffer first, which is never freed and
 *                  cannot be grown while the stream is being captured.
 *   cb64           int64[256]; byte i of entry e is int8(4 * codebook value i)
 *                  (test_decode_matmul.py:85).
 *   cb16           fp16[256][8]; the same table as real values (byte / 4).
 *   sign convention DMM_SIGN_SLOW: stored bit i -> weight i (i<7), parity -> weight 7
 *                  (decode_matmul_cuda.cu:50-53); DMM_SIGN_FAST: parity -> weight 0,
 *                  stored bit i -> weight i+1 (fast_decode_matmul_cuda.cu:52-53).
 * The fast kernels need every codebook byte to be congruent to 2 modulo 4 (true of the
 * E8P table and of tables drawn from {0.5,1.5,2.5,3.5}); the same assumption is built into
 * the reference's decode8weights.  A table that breaks it raises DMM_STATUS_BAD_CODEBOOK in
 * the device status word and the output of that call is undefined.
 */
#ifndef DMM_H_
#define DMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DMM_OK 0
#define DMM_ERR_NULL (-1)        /* a required pointer is NULL */
#define DMM_ERR_SHAPE (-2)       /* M < 1, N % 16 != 0, K % 32 != 0, or a size out of range */
#define DMM_ERR_ALIGN (-3)       /* a pointer is not 16-byte aligned */
#define DMM_ERR_ARG (-4)         /* unknown enum value */
#define DMM_ERR_WORKSPACE (-5)   /* caller-supplied workspace too small */
#define DMM_ERR_UNSUPPORTED (-6) /* shape outside what the chosen path implements */
#define DMM_ERR_LIMIT (-7)       /* size beyond the fixed scratch of dmm_f16_noalloc */

#define DMM_SIGN_SLOW 0
#define DMM_SIGN_FAST 1

#define DMM_LAYOUT_TILE 0 /* transpose_tile() layout, used by decode_matmul_cuda */
#define DMM_LAYOUT_FAST 1 /* uint32 [N/32][K/16][32] layout, used by fast_decode_matmul_cuda */

#define DMM_PATH_AUTO 0
#define DMM_PATH_GEMV 1       /* streaming kernel on warp-level MMAs, any M */
#define DMM_PATH_TCGEN05 2    /* tcgen05 + TMEM, decoded weights as fp16 operands, any M */
#define DMM_PATH_TCGEN05_F8 3 /* tcgen05 + TMEM, weights as fp6 and activations as exact fp8 planes,
                                 32 batch rows per pass over the weights; what DMM_PATH_AUTO takes */

/* what dmm_f16_fused reads as activations */
#define DMM_X_F16 0          /* fp16 [M, x_ld] */
#define DMM_X_F32 1          /* fp32 [M, x_ld], rounded to fp16 on the fly */
#define DMM_X_F32_SILU_MUL 2 /* fp32 [M, x_ld]: fp16(silu(x[:, k]) * x[:, x_gap + k]) */

/* launch flags (bit mask) */
#define DMM_FLAG_ACCUMULATE 1u /* out += result instead of out = result */
#define DMM_FLAG_PDL 2u        /* launch with programmatic stream serialization: the kernel's
                                  weight prefetch may overlap the tail of the previous kernel
                                  in the stream; activations are read only after it finished */

#define DMM_FLAG_ATOMIC 4u     /* tcgen05 paths: out += result by floating-point atomic adds (implies
                                  accumulate; zero `out` first for a plain product).  Saves the
                                  workspace round trip of partial sums at the end of the kernel; the
                                  summation order, hence the last bits of the result, is not fixed */

/* bits of the device status word */
#define DMM_STATUS_WAIT_TIMEOUT 1u /* a bounded device-side wait expired */
#define DMM_STATUS_BAD_CODEBOOK 2u /* codebook byte not congruent to 2 mod 4, or fp16 entry not k/4 */
#define DMM_STATUS_BAD_SMEM 4u     /* shared-memory carve-up did not fit */

/*
 * Integer family.  out[M,N] (int32) (+)= x[M,K] (int8) . decode(codes)[N,K]^T, exact.
 * Replaces the kernel and host wrapper of decode_matmul_cuda/decode_matmul_cuda.cu:68-234
 * (3-argument form: flags = 0) and of decode_matmul_cuda/fast_decode_matmul_cuda.cu:70-184
 * (4-argument, in-place accumulate form: flags = DMM_FLAG_ACCUMULATE, DMM_SIGN_FAST,
 * DMM_LAYOUT_FAST).  Accepts every M >= 1, N % 16 == 0 (N % 32 for the fast layout),
 * K % 32 == 0; the reference's extra limits (M % 8, K % 2048, K >= 4096) are gone.
 * Runs on the tcgen05 kernel (kind::i8 MMAs into int32 accumulators in tensor memory), 32 batch rows
 * per pass over the weights.
 * workspace may be NULL: the library then uses a per-device buffer it allocates on first
 * use; calls that can overlap on the GPU must pass distinct workspaces.
 */
int dmm_i8(const int8_t *x, const int16_t *codes, const int64_t *cb64, int32_t *out,
           int64_t M, int64_t N, int64_t K, int sign_convention, int layout, unsigned flags,
           void *workspace, size_t workspace_bytes, void *stream);

/*
 * fp16 family.  out[M,N] (fp32) (+)= scale * x[M,K] (fp16) . W[N,K]^T with
 * W = decode(codes)/4, fp32 accumulation.  The reference has no fp16 path; semantics are
 * its integer decode (test_decode_matmul.py:29-55) read as quarter units.
 * cb16 is fp16[256][8].  path: DMM_PATH_*.
 */
int dmm_f16(const void *x, const int16_t *codes, const void *cb16, float scale, float *out,
            int64_t M, int64_t N, int64_t K, int sign_convention, int layout, int path,
            unsigned flags, void *workspace, size_t workspace_bytes, void *stream);

/*
 * dmm_f16 with the operator's neighbours folded in (the elementwise steps that sit between two
 * quantised linear layers and that the reference leaves to the caller): the activation
 * loaders read the fp32 output of the previous layer and round it to fp16 themselves
 * (DMM_X_F32), or form silu(gate) * up of a fused gate/up output first (DMM_X_F32_SILU_MUL),
 * and DMM_FLAG_ACCUMULATE / DMM_FLAG_ATOMIC add the product onto a residual stream.  The
 * result equals running those steps separately in fp32 and calling dmm_f16.
 * x_ld = row stride of x in elements (>= K, multiple of 8); x_gap = offset of the second
 * operand for DMM_X_F32_SILU_MUL.  fp32 inputs take the small-batch tcgen05 path only.
 * zero_ptr / zero_count (optional): a float buffer that this kernel sets to zero once the
 * previous kernel of the stream has finished -- the output buffer of a LATER call that runs
 * with DMM_FLAG_ATOMIC, so that a chain of layers needs no memset between kernels.  The
 * buffer must not be read or written by this call or by the kernel right before it.
 * The reference has no counterpart: its operator starts at int8 activations
 * (decode_matmul_cuda.cu:186).
 */
int dmm_f16_fused(const void *x, int x_kind, int64_t x_ld, int64_t x_gap, const int16_t *codes,
                  const void *cb16, float scale, float *out, int64_t M, int64_t N, int64_t K,
                  int sign_convention, int layout, int path, unsigned flags, float *zero_ptr,
                  int64_t zero_count, void *workspace, size_t workspace_bytes, void *stream);

/*
 * Tensor-parallel form of dmm_f16_fused for row-parallel layers.  (No counterpart in the reference.)
 *
 * Every rank of a tensor-parallel group (one process per GPU) holds a K-shard of the weights and
 * produces a partial [M, N] product that has to be summed over the ranks.  Instead of a separate
 * all-reduce, the epilogue of this call adds its partial product to the SAME buffer on every rank:
 * peer_out[r] (r < n_peers <= 8) are device pointers to that buffer on each rank, this rank's own
 * included, the others mapped through NVLink peer memory (CUDA IPC / symmetric memory).  The adds
 * are system-scope atomic adds; once every rank has run the call and dmm_xrank_barrier has
 * completed, each rank's buffer holds its previous content plus the full product.
 * move_src / move_dst / move_count (optional): before any of that, move_dst[i] += move_src[i] and
 * move_src[i] = 0 on THIS rank (both local buffers) -- the residual stream changing from the buffer
 * the previous layers read to the buffer this layer adds to, so that no rank can add into a
 * buffer that a slower rank is still reading.  DMM_FLAG_ATOMIC | DMM_FLAG_ACCUMULATE are implied;
 * flags: DMM_FLAG_PDL only.  Everything else as dmm_f16_fused on the small-batch tcgen05 path.
 */
int dmm_f16_fused_tp(const void *x, int x_kind, int64_t x_ld, int64_t x_gap, const int16_t *codes,
                     const void *cb16, float scale, float *const *peer_out, int n_peers, int64_t M,
                     int64_t N, int64_t K, int sign_convention, unsigned flags, float *zero_ptr,
                     int64_t zero_count, float *move_src, float *move_dst, int64_t move_count, void *stream);

/*
 * Tensor-parallel step in the "slots" form: compute and collective in the matmul kernels themselves, one
 * NVLink traversal per row-parallel layer, no barrier and no separate reduction kernel.  (No counterpart
 * in the reference.)
 *
 * Every rank owns a slot array, float [2 parities][world][count] with count = M * N of the row-parallel
 * products, and `world` flag words followed by private words (at least 32 uint32 in all), both zero at the
 * start and both mapped on every rank (peer_slots[r], peer_flags[r]: the arrays of rank r; entry [rank] is
 * this rank's own).  Row-parallel layers are numbered by an epoch counter that the library keeps in the
 * flag array.
 *
 * dmm_f16_tp_produce: a row-parallel product.  The kernel accumulates the partial product into this rank's
 * own slot of the epoch's parity; the last CTA to finish copies the finished partial into this rank's slot
 * on every other rank with plain vector stores (one value per element and peer) and then raises this
 * rank's flag on every rank to the epoch number.  It also clears the own slot of the other parity.
 * dmm_f16_tp_consume: the column-parallel product that follows.  Its activation loaders wait, bounded
 * (DMM_STATUS_WAIT_TIMEOUT, dmm_set_wait_limit_ms), until the flags of all ranks show the epoch, and read
 * the activations as h_in + the slots of all ranks, summed in rank order (every rank gets the same bits);
 * the sum, the new residual stream, is also written to h_out ([M, K] fp32 like h_in; another buffer than
 * h_in).  Result: out (+)= scale * fp16(h_out) . W^T with atomic adds, as dmm_f16_fused with DMM_X_F32.
 * Ordering on the stream: a consume call must directly follow the produce call whose partial products it
 * reads (as the step of a transformer block does).  The consumer does not wait for that kernel as a whole:
 * this rank's own flag, raised after every CTA of the producer has finished, stands in for it, and the
 * consumer lets the kernel after it start only once it has seen the flags.
 * dmm_tp_finalize: h_out = h_in + slots of the last epoch, as a small kernel (end of a step).
 * Batch M <= 8.  flags: DMM_FLAG_PDL only.  Two slot parities suffice: a rank can start epoch e + 2 only
 * after every rank has finished reading epoch e.
 */
int dmm_f16_tp_produce(const void *x, int x_kind, int64_t x_ld, int64_t x_gap, const int16_t *codes, const void *cb16,
                       float scale, float *const *peer_slots, unsigned *const *peer_flags, int rank, int world,
                       int64_t M, int64_t N, int64_t K, int sign_convention, unsigned flags, void *stream);
int dmm_f16_tp_consume(const float *h_in, float *h_out, int64_t x_ld, const float *slots, const unsigned *flags_local,
                       int world, int64_t slot_count, const int16_t *codes, const void *cb16, float scale, float *out,
                       int64_t M, int64_t N, int64_t K, int sign_convention, unsigned flags, float *zero_ptr,
                       int64_t zero_count, void *stream);
int dmm_tp_finalize(const float *h_in, float *h_out, const float *slots, const unsigned *flags_local, int world,
                    int64_t count, void *stream);

/*
 * Barrier between the ranks of a tensor-parallel group, as a kernel on `stream`: returns (on the
 * device) once every rank has enqueued and reached the same barrier, which also makes the peer
 * adds of the dmm_f16_fused_tp calls before it visible.  peer_flags[r] (r < world <= 8) point to
 * an array of `world` uint32 on rank r, zero before the first barrier and owned by this function
 * afterwards; peer_flags[rank] is this rank's own array.  The wait is bounded
 * (DMM_STATUS_WAIT_TIMEOUT).  Every rank must call it the same number of times.
 */
int dmm_xrank_barrier(unsigned *const *peer_flags, int rank, int world, void *stream);

/*
 * One-shot all-reduce-and-add between the ranks of a tensor-parallel group, as a kernel on `stream`:
 * dst[i] += sum over ranks r of peer_src[r][i], i < count (count % 4 == 0), where peer_src[r] is the
 * buffer on rank r into which that rank's row-parallel layer accumulated its partial product
 * (plain dmm_f16_fused with DMM_FLAG_ATOMIC; this rank's own buffer included, the others mapped through
 * peer memory).  The kernel first runs the barrier of dmm_xrank_barrier (same peer_flags, same
 * rules; do not mix the two on one set of flags), then pulls the partials with coalesced loads over
 * NVLink and adds them in rank order, so every rank obtains the same bits.  zero_local (optional):
 * a local buffer of `count` floats that is cleared as well -- the partial buffer of the row-parallel
 * layer BEFORE this one, which every rank has finished reading once it has reached this barrier;
 * alternating two partial buffers this way needs no second barrier.
 */
int dmm_xrank_allreduce_add(float *dst, const float *const *peer_src, float *zero_local, int64_t count,
                            unsigned *const *peer_flags, int rank, int world, void *stream);

/*
 * A chain of dependent products in ONE launch.  (No counterpart in the reference.)
 *
 * ops[k] is one dmm_f16_fused product, out_k += scale_k * f(x_k) . W_k^T, where op k + 1 may
 * read what op k wrote (the next layer of a model).  Launched one by one, every layer pays
 * the launch, the table build and the filling and draining of the pipeline; in a chain the CTAs
 * stay resident, only the activation loaders wait at an op boundary (until every CTA has
 * finished the previous op), and the weight decoders are already working on the next op.
 * Rules: 2 <= n_ops <= DMM_CHAIN_MAX_OPS; batch M <= 8; tile layout; one codebook and sign
 * convention for all ops; results are ADDED to out_k with atomic adds (as DMM_FLAG_ATOMIC: out_k must
 * hold the value to add to, e.g. be cleared by the zero_ptr of an earlier op); flags: DMM_FLAG_PDL
 * only.  The CTAs wait for one another, so the kernel is launched cooperatively with one CTA per
 * SM: it needs the whole GPU, and two chains must not run at the same time on one device.
 * All device-side waits are bounded (DMM_STATUS_WAIT_TIMEOUT); after a timeout call
 * dmm_status() before the next chain (it also clears the chain's counters).
 */
#define DMM_CHAIN_MAX_OPS 8
typedef struct dmm_chain_op {
    const void *x;        /* activations of this op, see x_kind */
    int x_kind;           /* DMM_X_F16 / DMM_X_F32 / DMM_X_F32_SILU_MUL */
    int64_t x_ld, x_gap;  /* as in dmm_f16_fused */
    const int16_t *codes; /* tiled codes [N, K/8] */
    float scale;
    float *out;           /* [M, N] fp32, accumulated into */
    int64_t N, K;
    float *zero_ptr;      /* optional buffer cleared by this op (see dmm_f16_fused) */
    int64_t zero_count;
} dmm_chain_op;
int dmm_f16_chain(const dmm_chain_op *ops, int n_ops, const void *cb16, int64_t M, int sign_convention,
                  unsigned flags, void *stream);

/*
 * dmm_f16 for callers that must not allocate.  (No counterpart in the reference.)
 *
 * Some host programs cannot let a library call cudaMalloc on their behalf: a serving
 * process that has handed all of HBM to its own pool allocator (a later cudaMalloc simply
 * fails there), or a latency-critical loop that may not take the driver's allocator lock
 * or the implicit device synchronisation that comes with cudaMalloc and cudaFree.
 * dmm_f16 needs scratch memory for its stream-K
 * partial sums and, without a caller-supplied workspace, allocates it lazily.  This entry
 * point is the small-batch tcgen05 kernel (DMM_PATH_TCGEN05_F8) running on a scratch array
 * that is compiled into the library as a file-scope __device__ array instead: it calls no
 * cudaMalloc, no cudaFree and no allocating library routine, ever.
 *
 * Limits: M <= 8 and N <= 262144 (DMM_ERR_LIMIT beyond), tile layout only.  The array is
 * about 2.6 MB and every GPU that loads the library holds it until the process exits.
 * The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress); make that first call outside any stream capture.  With lazy module
 * loading (the CUDA default) the array and the kernel are placed in device memory at that first
 * call, so it must come before the host's own pool takes all of the device memory.
 * flags: DMM_FLAG_ACCUMULATE and DMM_FLAG_PDL only (DMM_ERR_ARG for any other bit).  All calls on
 * a device share the one array: two calls that can overlap on the GPU (different streams)
 * race on it and must be serialised by the caller.  Results equal dmm_f16 with
 * DMM_PATH_TCGEN05_F8.
 */
int dmm_f16_noalloc(const void *x, const int16_t *codes, const void *cb16, float scale, float *out,
                    int64_t M, int64_t N, int64_t K, int sign_convention, unsigned flags, void *stream);

/*
 * Decode only.  W_out[N,K] in logical (row-major) order: int8 (= 4 * weight) when
 * cb_is_f16 == 0 and cb is cb64, fp16 (= weight) when cb_is_f16 != 0 and cb is cb16.
 * Exposes decode8weights (decode_matmul_cuda.cu:45-65 / fast_decode_matmul_cuda.cu:46-67)
 * so that the decoded weights can be compared bit for bit.
 */
int dmm_decode(const int16_t *codes, const void *cb, int cb_is_f16, void *W_out, int64_t N,
               int64_t K, int sign_convention, int layout, void *stream);

/*
 * Hint for a sequence of products on one stream (the layers of a model): `codes` [N, K/8] (tile layout) is
 * the weight matrix of the product AFTER the next one this host thread enqueues.  The next dmm_f16 /
 * dmm_f16_fused / dmm_f16_fused_tp call of this thread consumes the hint: towards the end of its kernel
 * every CTA fetches into L2 (no other effect) the first codes that the same CTA of the following launch
 * will stream, so that the following launch does not begin with a DRAM round trip -- about a microsecond of
 * every launch's prologue at batch 1.  Purely a performance hint: results do not depend on it, a stale or
 * wrong hint only wastes a little bandwidth (the memory must be readable), NULL clears it.  The reference
 * has no counterpart (one product per call, decode_matmul_cuda.cu:178-234).
 */
int dmm_hint_next_weights(const int16_t *codes, int64_t N, int64_t K);

/*
 * How long the cross-rank waits of dmm_xrank_barrier / dmm_xrank_allreduce_add may last before they
 * give up, raise DMM_STATUS_WAIT_TIMEOUT and return (the kernel completes, the context stays usable):
 * `ms` milliseconds at about 2 GHz, 0 = the default of about a quarter of a second.  Applies to calls
 * enqueued afterwards, on every device.  A host that detects a lost rank on its own (heartbeat, store)
 * can keep the limit short so that the surviving ranks' streams drain quickly.  This replaces the
 * reference's only failure handling, gpuAssert -> exit() (decode_matmul_cuda.cu:35-42), for the
 * multi-GPU step, which the reference does not have.
 */
int dmm_set_wait_limit_ms(unsigned ms);

/* Bytes of workspace a call of dmm_i8 / dmm_f16 with these sizes needs (0 if none). */
size_t dmm_workspace_bytes(int64_t M, int64_t N, int64_t K);

/*
 * Reads and clears the status word of the current device (synchronises the device).
 * Replaces the reference's gpuAssert -> exit() (decode_matmul_cuda.cu:35-42).
 */
int dmm_status(unsigned *status_out);

/* Which path DMM_PATH_AUTO resolves to for this shape (one of the DMM_PATH_* values above). */
int dmm_select_path(int64_t M, int64_t N, int64_t K);

/* Number of kernels the library has launched in this process (all devices, all entry points). */
uint64_t dmm_launch_count(void);

/* Human-readable text for a return value of this API. */
const char *dmm_error_string(int code);

/* Library version, "major.minor". */
const char *dmm_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DMM_H_ */
