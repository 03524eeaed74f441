/*
 * gdn2_b200 -- C ABI of the Gated DeltaNet-2 forward / serving kernels for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers and sizes, launches on the given CUDA stream
 * (a cudaStream_t passed as void*, NULL = the legacy default stream), allocates nothing and
 * returns 0 or a negative gdn2_status. No C++ or framework types cross this boundary.
 *
 * Tensor conventions (those of the reference project's Python API):
 *   q, k, b : [B, S, HK, DK]  v, w : [B, S, H, DV]   element type `dtype`
 *   g       : [B, S, HK, DK]  fp32 natural-log decay, <= 0
 *   state   : [B, H, DK, DV]  fp32, contiguous
 *   o       : [B, S, H, DV]   element type `dtype`
 * H counts the value heads, HK the key heads, H a multiple of HK: value head h reads q, k, b, g of key head
 * h / (H / HK) (grouped-query heads). HK = H is the reference's layout, where its layer has already repeated
 * every key head H / HK times (gdn2/attention.py:295-297, 342); with HK < H the kernels index the key heads
 * instead and nothing is repeated in memory.
 * The [S, heads, D] block of one batch entry is contiguous; consecutive batch entries are
 * `in_batch_stride` (inputs) / `o_batch_stride` (o) TOKENS apart, counted in rows of heads*D elements
 * (pass S for a contiguous tensor). This lets a caller hand over a slice of a longer sequence --
 * the whole chunks to the chunkwise path, the ragged tail to gdn2_decode -- without copying it.
 *
 * The reference project has no native layer: its kernels are TileLang JIT factories called from
 * Python. Each function below names the reference Python interface whose device work it replaces
 * (paths relative to the reference project's root).
 */
#ifndef GDN2_B200_H_
#define GDN2_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GDN2_B200_ABI_VERSION 3

/* element type of q, k, v, b, w and o */
enum gdn2_dtype { GDN2_F32 = 0, GDN2_BF16 = 1, GDN2_F16 = 2 };

enum gdn2_status {
  GDN2_OK = 0,
  GDN2_ERR_NULL_POINTER = -1,   /* a required pointer is NULL */
  GDN2_ERR_BAD_SHAPE = -2,      /* a size is <= 0, S is not a multiple of 64, or a head dim is unsupported */
  GDN2_ERR_BAD_DTYPE = -3,      /* dtype is not a gdn2_dtype */
  GDN2_ERR_MISALIGNED = -4,     /* a pointer is not 16-byte aligned */
  GDN2_ERR_WORKSPACE = -5,      /* the workspace is smaller than gdn2_prefill_workspace_bytes() */
  GDN2_ERR_CUDA = -6,           /* a CUDA runtime call failed; see gdn2_last_cuda_error() */
  GDN2_ERR_DEVICE_WAIT = -7,    /* a kernel gave up on a bounded wait (reported by gdn2_check_device_status) */
  GDN2_ERR_UNSUPPORTED = -8,    /* valid arguments, but no kernel is built for this combination */
  GDN2_ERR_STATIC_LIMIT = -9    /* gdn2_prefill_static: the problem needs more than GDN2_STATIC_SCRATCH_BYTES */
};

/* Which kernel family runs the chunkwise prefill. AUTO picks the tcgen05 family when the shape
 * allows it (DK = DV = 128, bf16) and the SIMT family otherwise. The explicit values exist so the
 * two families can be cross-checked against each other; both are hand-written CUDA for sm_100a.
 * TCGEN05_SERIAL is the tcgen05 family with the scan forced to walk each (batch, head) in one
 * block; TCGEN05 (and AUTO) cut the sequence into segments scanned in parallel when a GPU holds so
 * few (batch, head) pairs that most SMs would idle (see gdn2_prefill_scan). Pass the SAME path to
 * gdn2_prefill_workspace_bytes, gdn2_chunk_prep and gdn2_prefill_scan of one problem. */
enum gdn2_prefill_path { GDN2_PATH_AUTO = 0, GDN2_PATH_SIMT = 1, GDN2_PATH_TCGEN05 = 2, GDN2_PATH_TCGEN05_SERIAL = 3 };

/* ABI version of the loaded library (== GDN2_B200_ABI_VERSION it was built with). */
int gdn2_abi_version(void);

/* Human-readable text for a gdn2_status. Never NULL. */
const char* gdn2_status_string(int status);

/* cudaError_t (as int) of the last failed CUDA call made by this library on the calling thread. */
int gdn2_last_cuda_error(void);

/*
 * n-token recurrent decode; `state` is read once, updated in place and written once.
 *   q,k,b [B,n,HK,DK]  v,w [B,n,H,DV]  g [B,n,HK,DK] fp32  state [B,H,DK,DV] fp32  o [B,n,H,DV]
 * n = 1 is the single-token step. Supported: DK <= 256, any DV >= 1, n >= 1. With DK = DV = 128 (the fast
 * kernels: 16-byte loads and bulk copies) every pointer must be 16-byte aligned, else GDN2_ERR_MISALIGNED.
 * Replaces decode_step_kernel / decode_multi_kernel and the device branch of gdn2_decode and
 * gdn2_decode_step (gdn2/inference.py:61-153, 199-303, 306-353, 156-196).
 */
int gdn2_decode(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                float* state, void* o, int64_t B, int64_t n, int64_t H, int64_t HK, int64_t DK, int64_t DV,
                int64_t in_batch_stride, int64_t o_batch_stride, float scale, int dtype, void* stream);

/*
 * Bytes of scratch the chunkwise prefill needs for a [B,S,H,DK,DV] problem (S a multiple of 64).
 * Returns 0 for an unsupported combination. `path` is a gdn2_prefill_path.
 */
size_t gdn2_prefill_workspace_bytes(int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK, int64_t DV, int dtype,
                                    int path);

/*
 * Byte offsets of the record arrays inside the workspace, for tools and tests that inspect the
 * intermediates: out8 = { WQ, AQK, KG^T, U^T, gamma_last, flags, segment records, total bytes }.
 * WQ, AQK, KG^T, gamma_last and the flags are indexed by KEY chunk-head (b*HK + hk)*(S/64) + n, U^T by value
 * chunk-head (b*H + h)*(S/64) + n. Tensor-core family (DK = DV = 128, bf16):
 *   WQ    32 KiB  bf16 [dk/8][128 rows][8]: rows 0..63 = W of token r, rows 64..127 = scale*q*gamma of token r-64
 *   AQK    8 KiB  fp16 [s/8][64 r][8]:  256 * Aqk[r, s], lower triangular including the diagonal
 *   KG^T  16 KiB  fp16 [t/8][128 dk][8]: 256 * k[t, dk] * gamma_last[dk] / gamma[t, dk]
 *   U^T   16 KiB  fp16 [t/8][128 dv][8]: U[t, dv] / 256
 *   gamma_last 512 B fp32 [dk]
 * SIMT family: the same images with 4-byte elements ([x/4][rows][4]) and no scaling.
 * No counterpart in the reference, whose intermediates are separate tensors (gdn2/forward.py:756-829).
 */
int gdn2_prefill_workspace_layout(int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK, int64_t DV, int dtype,
                                  int path, int64_t* out8);

/*
 * Number of sequence segments gdn2_prefill_scan cuts this problem into (1 = one block per (batch, head)
 * walks the whole sequence; 0 for an unsupported combination). A caller that overlaps the two stages of
 * its own sequence segments on two streams uses this to see that the scan already fills the GPU.
 * No counterpart in the reference.
 */
int gdn2_prefill_scan_segments(int64_t B, int64_t S, int64_t H, int64_t DK, int64_t DV, int dtype, int path);

/*
 * Kernels gdn2_prefill_scan launches for this problem without chunk_states: 1 (one walk), 3 (first pass, chaining
 * of the segment records, redo pass) or 4 (the same behind the decay check of a guarded cut); 0 for an
 * unsupported combination. For callers that account for their launches. No counterpart in the reference.
 */
int gdn2_prefill_scan_launches(int64_t B, int64_t S, int64_t H, int64_t DK, int64_t DV, int dtype, int path);

/*
 * Chunk-local stage of the chunkwise forward (chunk = 64 tokens): cumulative log2 decay, the
 * intra-chunk matrices Aqk / Akk, the (I + Akk)^-1 solve and the WY factors W, U, KG, plus the
 * decayed queries, written into `workspace` in the operand layout the scan consumes.
 * Replaces cumsum_kernel, intra_diag_kernel, inter_blocks_kernel, solve_kernel, wy_kernel and their
 * driver wy_stages (gdn2/forward.py:65-535, 756-829).
 */
int gdn2_chunk_prep(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                    void* workspace, size_t workspace_bytes, int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK,
                    int64_t DV, int64_t in_batch_stride, float scale, int dtype, int path, void* stream);

/*
 * Sequential state scan over chunks fused with the output: per chunk Un = U - W S,
 * o = Qg S + tril(Aqk) Un, S <- diag(gamma_C) S + KG^T Un, with the fp32 state resident on chip.
 *   initial_state  [B,H,DK,DV] fp32 or NULL (zeros)
 *   final_state    [B,H,DK,DV] fp32 or NULL (not written)
 *   chunk_states   [B,S/64,H,DK,DV] fp32 or NULL; when given, the state entering every chunk is stored
 * Replaces prefill_scan_kernel (gdn2/inference.py:356-479) and, with chunk_states, the
 * state_kernel + output_kernel pair of the training-style forward (gdn2/forward.py:538-727).
 *
 * Few (batch, head) pairs (tcgen05 family, no chunk_states; B*H <= 28 and 24 chunks or more: always; B*H <= 72 and
 * 48 chunks or more: "guarded", only when a check of the decay on the device finds that a segment forgets the
 * state entering it): the sequence is cut into segments. Every segment is scanned from a zero state while a second block
 * accumulates the segment's state-transition matrix; a small kernel chains the segments' affine maps
 * and a last launch redoes, from the true entering state, the leading chunks of each segment that the
 * entering state still reaches. The result equals the one-block walk up to the rounding of the state
 * hand-over (below 1e-6 of the state); the form used is reported by gdn2_prefill_scan_segments.
 */
int gdn2_prefill_scan(const void* workspace, size_t workspace_bytes, const float* initial_state, void* o,
                      float* final_state, float* chunk_states, int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK,
                      int64_t DV, int64_t o_batch_stride, int dtype, int path, void* stream);

/*
 * gdn2_prefill_scan (without chunk_states) in two calls, for a caller that has work which needs only the final state
 * -- the decode of a ragged tail -- and wants it to run beside the rest of the scan on another stream:
 *   part 1  everything up to the final state: for a cut scan the decay check, the first pass and the chaining of
 *           the segments (final_state is complete when it ends, the outputs of the leading chunks of every
 *           segment are not yet); for a scan that is not cut, the whole scan;
 *   part 2  what is left: the correction pass of a cut scan (initial_state and final_state are ignored), else
 *           nothing.
 * Both parts take the same arguments. No counterpart in the reference.
 */
int gdn2_prefill_scan_part(const void* workspace, size_t workspace_bytes, const float* initial_state, void* o,
                           float* final_state, int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK, int64_t DV,
                           int64_t o_batch_stride, int dtype, int path, int part, void* stream);

/*
 * The whole of gdn2_prefill (gdn2/inference.py:482-555) in one call, for callers that count host microseconds:
 * gdn2_chunk_prep + gdn2_prefill_scan on the floor(S/64)*64 leading tokens and gdn2_decode on the ragged tail
 * (S need not be a multiple of 64), the state chained through final_state (written even without a tail; must not be
 * initial_state unless S < 64).
 *   workspace     gdn2_prefill_workspace_bytes(B, floor(S/64)*64, ...) bytes; NULL is accepted when S < 64
 *   side_stream   NULL, or a second stream of the same device: when the scan is cut into segments the tail's decode,
 *                 which needs only the final state, runs there beside the scan's correction pass; `stream` is ordered
 *                 after it when the call returns
 * Results are those of the three calls made one after the other. No counterpart in the reference as ONE function:
 * its gdn2_prefill is the same sequence in Python.
 */
int gdn2_prefill_ragged(const void* q, const void* k, const void* v, const float* g, const void* b, const void* w,
                        const float* initial_state, void* o, float* final_state, void* workspace, size_t workspace_bytes,
                        int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK, int64_t DV, int64_t in_batch_stride,
                        int64_t o_batch_stride, float scale, int dtype, int path, void* side_stream, void* stream);

/*
 * gdn2_prefill_scan with the layer's gated RMSNorm as the epilogue of the output rows:
 *   o[b,t,h,:] <- o * rsqrt(mean(o^2) + eps) * weight * silu(gate[b,t,h,:]),
 * evaluated on the rows as they leave the chip (rounded to `dtype` first, as the separate kernel would read
 * them), so the normalised rows are written once and the plain ones never. The gate of o[b,t,h,c] is read at
 * gate[(b * gate_batch_stride + t) * gate_row_stride + h*DV + c]: pass the o_gate columns of the layer's
 * projection buffer without copying them. Tensor-core family only (DK = DV = 128, bf16; otherwise
 * GDN2_ERR_UNSUPPORTED: use gdn2_prefill_scan + gdn2_layer_back). norm == NULL is gdn2_prefill_scan.
 * Replaces _GatedRMSNorm after the attention call (gdn2/attention.py:218-229, 354-355).
 */
typedef struct gdn2_gated_norm {
  const void* gate;            /* `dtype`, 16-byte aligned, gate_row_stride a multiple of 8 */
  const void* weight;          /* [DV] `dtype` */
  int64_t gate_row_stride;     /* elements between tokens */
  int64_t gate_batch_stride;   /* tokens between batch entries */
  float eps;
} gdn2_gated_norm;
int gdn2_prefill_scan_gated_norm(const void* workspace, size_t workspace_bytes, const float* initial_state, void* o,
                                 float* final_state, int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK,
                                 int64_t DV, int64_t o_batch_stride, int dtype, int path, const gdn2_gated_norm* norm,
                                 void* stream);

/*
 * Chunk-parallel output from stored chunk states: o = Qg h_n + tril(Aqk) Un_n with
 * Un_n = U - W h_n, one thread block per (chunk, batch, head). Needs the workspace of
 * gdn2_chunk_prep and the chunk_states of gdn2_prefill_scan.
 * Replaces output_kernel (gdn2/forward.py:644-727).
 */
int gdn2_chunk_output(const void* workspace, size_t workspace_bytes, const float* chunk_states, void* o,
                      int64_t B, int64_t S, int64_t H, int64_t HK, int64_t DK, int64_t DV, int64_t o_batch_stride,
                      int dtype, int path, void* stream);

/*
 * Kernels with bounded waits record a non-zero word when a wait runs out. This copies the word
 * for the current device to the host (synchronising `stream` first), clears it and returns
 * GDN2_OK or GDN2_ERR_DEVICE_WAIT. `detail` (may be NULL) receives the raw word.
 */
int gdn2_check_device_status(void* stream, uint32_t* detail);

/*
 * Self-test of the tcgen05 / TMEM / bulk-copy building blocks on tiny fixed operands
 * (one 128x128x64 bf16 and one tf32 product through shared-memory descriptors, a TMEM round trip).
 * `out` receives 4*128*128 fp32 results (the bf16 product, the tf32 product, 2*tf32+1 after a TMEM
 * store/load round trip, and the bf16 product again with A read from tensor memory); `a` and `bt` are [128,64] fp32 row-major inputs (A, and B transposed).
 * No counterpart in the reference.
 */
int gdn2_selftest_mma(const float* a, const float* bt, float* out, void* stream);

/*
 * Self-test of the failure path: one small block waits, with a limit of `limit_cycles` SM clock cycles
 * (1 .. 2e9), on a barrier that nothing ever satisfies. The wait gives up, the block returns normally, the
 * device stays usable, and the next gdn2_check_device_status reports GDN2_ERR_DEVICE_WAIT with bit 31
 * of the detail word set. `gave_up` (device pointer to an int, may be NULL) is incremented once per
 * thread whose wait ran out (64 threads). No counterpart in the reference.
 */
int gdn2_selftest_wait(int64_t limit_cycles, int* gave_up, void* stream);

/*
 * Whole-chunk prefill that allocates nothing and asks the caller for no workspace: the chunk-local
 * stage and the fused scan of gdn2_chunk_prep + gdn2_prefill_scan, exchanging their intermediates
 * through a fixed scratch array built into the library. It has no counterpart in the reference.
 *
 * It exists for callers that cannot obtain device memory at call time: a plugin inside a serving
 * engine that has already given all free HBM to its own pool, a latency-critical loop that cannot
 * afford the device-wide synchronisation cudaMalloc / cudaFree imply, or a host that only lends
 * pre-registered input and output buffers. Such callers still pass q, k, v, g, b, w,
 * initial_state (may be NULL), o and final_state (may be NULL) exactly as for the two-call form;
 * S must be a multiple of 64 (send a ragged tail through gdn2_decode).
 *
 * Limit: the problem's scratch, gdn2_prefill_workspace_bytes(B, S, H, DK, DV, dtype, AUTO), must
 * not exceed GDN2_STATIC_SCRATCH_BYTES -- about 450 chunk-heads (B * H * S/64) at DK = DV = 128 in
 * bf16. Larger problems return GDN2_ERR_STATIC_LIMIT and launch nothing; split them over batch,
 * heads or sequence segments, or use the two-call form. Every GPU that loads the library holds the
 * array until the process exits.
 *
 * The first call on each device resolves the array's device address (cudaGetSymbolAddress) with
 * that device current; make that first call outside any stream capture. That first call is also the
 * moment the CUDA driver brings the library's device image -- and with it the 32 MiB array -- into
 * device memory (module loading is lazy by default), so it is a warm-up that DOES take device memory:
 * make it at start-up, before the rest of HBM is handed to a pool (a tiny problem is enough); if it
 * comes later and no memory is left it returns GDN2_ERR_CUDA. Every later call on that device
 * allocates nothing. All calls on a device
 * share the one array, which keeps whatever the previous call left in it: each call rewrites every
 * record it later reads, so nothing needs clearing, but two calls that overlap on the GPU (different
 * streams, or concurrent host threads) race on it -- serialise them.
 */
#define GDN2_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
int gdn2_prefill_static(const void* q, const void* k, const void* v, const float* g, const void* b,
                        const void* w, const float* initial_state, void* o, float* final_state,
                        int64_t B, int64_t S, int64_t H, int64_t DK, int64_t DV,
                        int64_t in_batch_stride, int64_t o_batch_stride, float scale, int dtype,
                        void* stream);

/*
 * Element-wise stages of the GatedDeltaNet2 layer, fused. The caller computes ONE projection buffer
 * proj [B, S, NP] = x W_cat^T whose columns hold, at the given offsets, the q, k, v, b, w, f and o_gate
 * projections (q, k, b, f: HK*DK columns each; v, w, o_gate: H*DV columns each).
 *
 * gdn2_layer_front writes the six kernel inputs in the layout of gdn2_prefill / gdn2_decode:
 *   q, k, b [B, S, HK, DK] and v, w [B, S, H, DV] in `dtype`, g [B, S, HK, DK] fp32 (one copy per key head: the
 *   attention kernels index key heads, gdn2/attention.py:295-297's repeat_interleave is not materialised), with
 *   q, k = l2norm(silu(conv(proj_q,k)))  v = silu(conv(proj_v))  (depthwise causal convolution of K taps:
 *   conv_weight [2*HK*DK + H*DV, K], conv_bias [same] or NULL, channels ordered q | k | v; K = 0 skips it),
 *   b = erase_scale * sigmoid(proj_b)  w = sigmoid(proj_w)  g = -exp(A_log[hk]) * softplus(proj_f + dt_bias[hk]),
 *   conv_state [B, 2*HK*DK + H*DV, K-1] (or NULL = zeros)
 *   supplies the columns before the first token; new_conv_state (or NULL) receives the last K-1
 *   pre-convolution columns. new_conv_state may be conv_state itself (the cache updated in place) only for
 *   S = 1 with 16-bit `dtype`, DK = DV = 128, K = 4 and NP and the column offsets multiples of 4: there one
 *   kernel reads a channel's old columns and writes its new ones from the same thread. In every other case the
 *   two must not overlap. A_log [HK] and dt_bias [HK, DK] are in `dtype`.
 * gdn2_layer_back writes out [B*S, H*DV] = rmsnorm_per_head(o) * norm_weight[DV] * silu(proj_o_gate).
 * Replaces the operator chains of _ShortConv, F.normalize, the gate expressions, repeat_interleave and
 * _GatedRMSNorm (gdn2/attention.py:186-229, 290-297, 323-340, 352-354).
 */
typedef struct gdn2_layer_front_args {
  const void* proj;            /* [B, S, NP] */
  const void* conv_state;      /* [B, CC, K-1] or NULL */
  const void* conv_weight;     /* [CC, K] */
  const void* conv_bias;       /* [CC] or NULL */
  const void* A_log;           /* [HK] */
  const void* dt_bias;         /* [HK, DK] */
  void* q; void* k; void* v; float* g; void* b; void* w;
  void* new_conv_state;        /* [B, CC, K-1] or NULL */
  int64_t B, S, H, HK, DK, DV, K, NP;
  int64_t off_q, off_k, off_v, off_b, off_w, off_f;
  float erase_scale;
} gdn2_layer_front_args;

int gdn2_layer_front(const gdn2_layer_front_args* args, int dtype, void* stream);
int gdn2_layer_back(const void* o, const void* proj, const void* norm_weight, void* out, int64_t BS, int64_t H,
                    int64_t DV, int64_t NP, int64_t off_gate, float eps, int dtype, void* stream);

/*
 * Output projection of a head-parallel layer fused with its all-reduce, for decode-sized inputs (1..8 token
 * rows): out [rows, hidden] = sum over the `world` ranks of x_r [rows, K] * weight_r [hidden, K]^T, the same
 * bits on every rank. One launch per rank and call; all ranks must make the same sequence of calls.
 *
 * The ranks exchange their fp32 partial sums through an exchange buffer that every rank allocates with
 * gdn2_oproj_reduce_buffer_bytes() bytes, zeroes ONCE before the first call, and maps into its peers' address
 * spaces (CUDA IPC, cuMem handles or a symmetric-memory allocator; ordinary peer loads and stores over NVLink,
 * no multicast). peer_slots[r] is rank r's buffer as seen from THIS rank (its own buffer at index `rank`),
 * peer_flags[r] the same buffer plus the flags offset the size query reports; both arrays live in device memory.
 * `epochs` is a local device array of hidden / 32 uint32, zeroed once. A rank that waits longer than
 * `wait_cycles` SM clock cycles (0 = about 0.1 s) for a peer's partial gives up: the call still completes,
 * gdn2_check_device_status then reports GDN2_ERR_DEVICE_WAIT (detail bit 30) and `out` is not to be used.
 * world == 1 degenerates to the plain product (peer arrays may be NULL).
 * Limits: hidden a multiple of 32; K a multiple of 8 (4 for fp32); rows * K elements at most 64 KiB.
 * Replaces F.linear(o_proj) followed by an all-reduce in the sharded form of gdn2/attention.py:354-356;
 * the reference itself has no multi-GPU code.
 */
typedef struct gdn2_oproj_reduce_args {
  const void* x;                 /* [rows, K] */
  const void* weight;            /* [hidden, K], this rank's columns of o_proj.weight */
  void* out;                     /* [rows, hidden] */
  void* const* peer_slots;       /* device array [world] */
  uint32_t* const* peer_flags;   /* device array [world] */
  uint32_t* epochs;              /* device array [hidden / 32], local */
  int64_t rows, K, hidden;
  int rank, world;
  int64_t wait_cycles;
} gdn2_oproj_reduce_args;

/* Bytes of one rank's exchange buffer; *flags_offset (may be NULL) receives the byte offset of its flag array. */
size_t gdn2_oproj_reduce_buffer_bytes(int64_t world, int64_t hidden, size_t* flags_offset);
int gdn2_oproj_reduce(const gdn2_oproj_reduce_args* args, int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* GDN2_B200_H_ */
