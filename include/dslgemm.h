/*
 * libdslgemm - C ABI of the B200 (sm_100a) quantised-GEMM library.
 *
 * Every entry point takes raw device pointers and an explicit CUDA stream (passed as
 * void*, i.e. a cudaStream_t), allocates nothing, never synchronises, and returns
 *     0   success (work enqueued on the stream)
 *   < 0   invalid argument (DSL_ERR_*), nothing enqueued
 *   > 0   a cudaError_t value from the launch
 * Kernels that wait on hardware barriers bound every wait; a kernel that gave up ORs a
 * DSL_ST_* bit into the caller's status word (device memory, may be NULL) and exits
 * cleanly, so the context stays usable.  Read the word after synchronising the stream.
 *
 * Operand conventions: A is [M, K] row-major (K contiguous); weights are K-major
 * [N, K] (or [G, N, K] for grouped GEMM).  FP4 operands hold two e2m1 values per byte,
 * low nibble = even k.  Block-scale bytes use the 512-byte tile layout
 *   tile(rt, kt) at (rt * ceil(nblk/4) + kt) * 512,  byte(r, c) at (r%32)*16 + (r/32)*4 + c
 * for 128 rows x 4 K-blocks per tile; dsl_sf_bytes() gives the buffer size.
 */
#ifndef DSLGEMM_H_
#define DSLGEMM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { DSL_F32 = 0, DSL_BF16 = 1, DSL_F16 = 2 };                       /* input / output dtypes */
enum { DSL_FP8_PER_TENSOR = 0, DSL_FP8_GROUP_1X128 = 1, DSL_FP8_BLOCK_128X128 = 2 };
enum { DSL_FP4_NV = 0, DSL_FP4_MX = 1 };                                /* NVFP4 / MXFP4 */

enum {
    DSL_ERR_NULL = -1,        /* required pointer is NULL */
    DSL_ERR_SHAPE = -2,       /* size negative, too large, or not a multiple the format needs */
    DSL_ERR_ALIGN = -3,       /* pointer or leading dimension not 16-byte aligned */
    DSL_ERR_ENUM = -4,        /* unknown dtype / mode / format */
    DSL_ERR_DRIVER = -5,      /* the CUDA driver's tensor-map encoder is unavailable or refused */
    DSL_ERR_TOO_LARGE = -6    /* beyond a stated fixed capacity */
};
enum {
    DSL_ST_TIMEOUT_PRODUCER = 1, DSL_ST_TIMEOUT_MMA = 2, DSL_ST_TIMEOUT_EPILOGUE = 4, DSL_ST_TIMEOUT_TEST = 8
};

#define DSL_MAX_GROUPS 1024

const char* dsl_version(void);

/* Bytes of the tiled scale-factor buffer for `rows` x `nblk` scale bytes (one group). */
size_t dsl_sf_bytes(long long rows, long long nblk);
/* Same for ragged row groups, each padded to whole 128-row tiles: upper bound that needs
 * no knowledge of the split - (ceil(rows/128) + groups) tiles. */
size_t dsl_sf_bytes_grouped(long long rows, long long nblk, int groups);

/*
 * FP8 E4M3 quantisation.  Replaces quantize_to_fp8_kernel (cuda/gemm/fp8_gemm.cu:119-144)
 * and extends it to 1x128 K-groups and 128x128 blocks.
 *   x          [rows, cols] of `dtype`, contiguous, 16-byte aligned; cols % 16 == 0 for the grouped modes
 *   scale_io   per-tensor: 1 float (written, or read when scale_given != 0)
 *              1x128: [rows, ceil(cols/128)] written;  128x128: [ceil(rows/128), ceil(cols/128)] written
 *   q_out      [rows, cols] bytes
 *   ws         4 bytes of scratch (per-tensor amax)
 */
int dsl_quant_fp8(const void* x, int dtype, long long rows, long long cols, int mode, float* scale_io,
                  int scale_given, uint8_t* q_out, void* ws, void* stream);

/*
 * FP4 e2m1 quantisation with block scales.  Replaces quantize_fp32_to_nvfp4
 * (cuda/gemm/fp4_gemm.cu:50-90) for the two standard formats:
 *   DSL_FP4_NV  one unsigned-E4M3 scale per 16 K-elements + fp32 global scale (cols % 32 == 0)
 *   DSL_FP4_MX  one E8M0 scale per 32 K-elements                               (cols % 32 == 0)
 *   gs_io      NVFP4 global scale: written (amax/2688), or read when gs_given != 0; unused for MX
 *   q_out      [rows, cols/2] bytes;  sf_out tiled scale bytes (dsl_sf_bytes / _grouped)
 *   group_offsets  NULL, or int32[groups+1] device array of row offsets (ragged expert
 *              groups, each starting a fresh 128-row scale tile); groups <= DSL_MAX_GROUPS
 *   ws         4 bytes of scratch
 */
int dsl_quant_fp4(const void* x, int dtype, long long rows, long long cols, int format, float* gs_io,
                  int gs_given, uint8_t* q_out, uint8_t* sf_out, const int* group_offsets, int groups,
                  void* ws, void* stream);

/*
 * NVFP4 with one global scale per row ("per token"): gs_out[m] = amax of row m / 2688 (1 for an all-zero row), block
 * scales and values as in dsl_quant_fp4 with that row's global scale.  Same outputs and layouts as dsl_quant_fp4 plus
 * gs_out [rows] fp32.  Because a row needs nothing but itself, this is ONE pass over x (dsl_quant_fp4 with a dynamic
 * tensor-wide scale is an amax pass plus a quantise pass); the GEMM applies gs_out as dsl_epilogue.row_scale with
 * scale_a = 1.  cols <= DSL_PER_TOKEN_MAX_COLS (a row is held in one CTA's registers).  Extends quantize_fp32_to_nvfp4
 * (cuda/gemm/fp4_gemm.cu:50-90), whose scale is likewise local (per 32 elements).
 */
#define DSL_PER_TOKEN_MAX_COLS 32768
int dsl_quant_fp4_per_token(const void* x, int dtype, long long rows, long long cols, float* gs_out, uint8_t* q_out,
                            uint8_t* sf_out, const int* group_offsets, int groups, void* stream);

/* Byte-matrix transpose [R, C] -> [C, R]: turns the reference's [K, N] weight layout
 * (cuda/gemm/fp8_gemm.cu:29-35, B[k*N+n]) into the K-major [N, K] the tensor cores read. */
int dsl_transpose_u8(const uint8_t* in, uint8_t* out, int R, int C, void* stream);

enum { DSL_ACT_NONE = 0, DSL_ACT_SWIGLU = 1, DSL_ACT_GEGLU = 2 };
enum { DSL_OUT_NVFP4 = 3 };   /* a value of dsl_epilogue.out_dtype besides DSL_F32 / DSL_BF16 */

/* Epilogue description shared by the GEMM entry points.
 *   out = acc * scale_a * scale_b [* row_scale[m]] [* col_scale[g*N+n]]
 * scale_x is *scale_x_dev when that pointer is non-NULL, else scale_x_host.
 * Zero the struct before filling it in: every field added after `workspace_bytes` means "off" when 0 / NULL.
 * With a workspace, dense problems with at most 128 rows go to the weight-streaming kernel (all SMs
 * stream equal shares of B; shared tiles are summed in ascending K order), and other dense problems
 * that would occupy less than half of the SMs are cut along K into up to 8 slices summed in order. */
typedef struct {
    float scale_a_host, scale_b_host;
    const float* scale_a_dev;
    const float* scale_b_dev;
    const float* row_scale;     /* [M_total] or NULL: per-token rescale */
    const float* col_scale;     /* [G, N]   or NULL: per-channel rescale */
    int out_dtype;              /* DSL_F32 or DSL_BF16 */
    void* workspace;            /* optional scratch (16-byte aligned) for partial sums along K, or NULL */
    size_t workspace_bytes;     /* its size: dsl_workspace_bytes() says what a problem can put to use (less is
                                   allowed and only slower).  The first 64 KiB are a header in which only the
                                   weight-streaming kernel's arrival words ever live; the buffer need not be cleared,
                                   and launches that may overlap on the GPU need separate buffers */
    int b_is_static;            /* non-zero: B and its scale bytes were complete before the kernel that precedes
                                   this call in the stream was launched (a pre-packed weight).  The weight-streaming
                                   kernel is launched with programmatic stream serialisation and then starts
                                   fetching B while that predecessor (e.g. the activation quantiser) still runs;
                                   A, its scales and every output are touched only after the predecessor is done. */
    int activation;             /* DSL_ACT_NONE, or DSL_ACT_SWIGLU / DSL_ACT_GEGLU: the GEMM's columns are (gate, up) pairs - column 2j
                                   is gate_j, column 2j+1 is up_j, i.e. the weight rows were interleaved when it was
                                   packed - and C is [M_total, N/2] with C[m,j] = silu(gate) * up computed in fp32 on
                                   the fully scaled values, silu(x) = x / (1 + exp(-x)); ldc >= N/2.  Fuses the
                                   reference's swiglu (cuda/activations/fused_gated_activations.cu:27-29,75-90) into
                                   the epilogue of the gate/up projection.  GEGLU: gelu(gate) * up with the tanh form
                                   of the same file (:32-37, :92-105). */
    void* out_sf;               /* out_dtype == DSL_OUT_NVFP4 only: the result (after the activation, if any) is
                                   quantised in the epilogue exactly as dsl_quant_fp4 would quantise it with the global
                                   scale given here: C receives packed e2m1 bytes [M_total, Nout/2] (row pitch ldc/2
                                   bytes, ldc % 16 == 0, Nout % 16 == 0) and out_sf the scale tiles (dsl_sf_bytes /
                                   dsl_sf_bytes_grouped; zero-filled by the caller, rows of a ragged group start fresh
                                   tiles as for A).  The next GEMM can consume C / out_sf as its A / sfa directly.
                                   Served by dsl_gemm_fp4, dsl_gemm_fp8 and dsl_gemm_bf16 (not the group-scaled FP8 GEMM). */
    float out_gs_host;          /* global scale of the quantised result ... */
    const float* out_gs_dev;    /* ... overridden by this device scalar when non-NULL */
    int act_scale_per_token;    /* dsl_linear with an NVFP4 weight only: quantise the activations with per-token global
                                   scales (dsl_quant_fp4_per_token, one pass) and apply them as the per-token rescale;
                                   row_scale must then be NULL */
} dsl_epilogue;

/*
 * Bytes of dsl_epilogue.workspace that the GEMM entry point `op` can put to use for a dense M x N x K
 * problem on the CURRENT device (it asks for the device's SM count), header included; 0 when the kernels
 * that serve the problem need no scratch (large M, row groups, decode shapes whose partial tiles are
 * combined inside thread-block clusters, the group-scaled FP8 GEMM).  Decode shapes with more 128-column
 * tiles than SMs take 2 partial tiles of TOK x 128 floats per CTA (TOK = 16 or 32 tokens); other
 * problems that would leave more than half of the SMs idle take up to 8 K-slices of M x N floats.
 */
enum { DSL_OP_GEMM_FP8 = 0, DSL_OP_GEMM_BF16 = 1, DSL_OP_GEMM_FP4_NV = 2, DSL_OP_GEMM_FP4_MX = 3, DSL_OP_GEMM_FP8_GROUPWISE = 4 };
size_t dsl_workspace_bytes(int op, long long M, int N, int K, int groups);

/*
 * Dense / grouped FP8 E4M3 GEMM, per-tensor scales: C[m,n] = sum_k A[m,k] B[n,k] * scale_a * scale_b.
 * Replaces fp8_gemm_per_tensor (cuda/gemm/fp8_gemm.cu:102-108) and the registered Triton
 * fp8_gemm (triton/gemm/gemm_kernels.py:104-122).  K % 16 == 0.
 * Grouped form (group_offsets != NULL): A is [M_total, K] with group g owning rows
 * offsets[g]..offsets[g+1]; B is [G, N, K]; C is [M_total, N]
 * (variable-size groups of cuda/gemm/grouped_gemm.cu:79-104, GemmProblem at :27-32).
 */
int dsl_gemm_fp8(const uint8_t* A, const uint8_t* B, void* C, long long ldc, long long M_total, int N, int K,
                 const int* group_offsets, int groups, const dsl_epilogue* ep, uint32_t* status, void* stream);

/*
 * Dense / grouped BF16 GEMM, fp32 accumulate (same conventions as dsl_gemm_fp8, operands bf16).
 * Replaces the registered grouped_gemm (triton/gemm/gemm_kernels.py:164-182; fixed-size groups of
 * cuda/gemm/grouped_gemm.cu:36-75 when all groups have equal rows) for unquantised inputs.  K % 8 == 0.
 */
int dsl_gemm_bf16(const void* A, const void* B, void* C, long long ldc, long long M_total, int N, int K,
                  const int* group_offsets, int groups, const dsl_epilogue* ep, uint32_t* status, void* stream);

/*
 * FP8 GEMM with fp32 group scales along K (G = 128):
 *   C[m,n] = sum_g (sum_{k in g} A[m,k] B[n,k]) * sa[m,g] * sb[g,n]
 * Replaces fp8_gemm_groupwise (cuda/gemm/fp8_gemm.cu:69-99,110-116).  sa is [M_total, K/128];
 * sb is [G, K/128, N] per-column scales when sb_block == 0 (the reference layout), or
 * [G, ceil(N/128), K/128] 128x128 block scales when sb_block != 0.  K % 128 == 0.
 */
int dsl_gemm_fp8_groupwise(const uint8_t* A, const uint8_t* B, const float* sa, const float* sb, int sb_block,
                           void* C, long long ldc, long long M_total, int N, int K, const int* group_offsets,
                           int groups, const dsl_epilogue* ep, uint32_t* status, void* stream);

/*
 * Dense / grouped block-scaled FP4 GEMM on packed e2m1 operands.
 * Replaces fp4_gemm (cuda/gemm/fp4_gemm.cu:95-146) for the two standard formats; for NVFP4 the
 * epilogue's scale_a/scale_b carry the two global scales.  sfa / sfb are tiled scale bytes
 * (sfa over A's rows - with ragged groups each group starts a fresh tile; sfb over [G][N]
 * with ceil(N/128) tiles per group).  K % 32 == 0.
 */
int dsl_gemm_fp4(const uint8_t* A, const uint8_t* B, const uint8_t* sfa, const uint8_t* sfb, int format, void* C,
                 long long ldc, long long M_total, int N, int K, const int* group_offsets, int groups,
                 const dsl_epilogue* ep, uint32_t* status, void* stream);

/*
 * One step of the hot path in a single call: quantise / scale-pack the activations x [M, K] (`x_dtype`) in the
 * format of the packed weight and multiply, C[M, N] = x_q @ W^T with the epilogue of the matching dsl_gemm_*
 * entry point.  Replaces the reference's per-call sequence quantise A, quantise B, GEMM
 * (cuda/gemm/fp8_gemm.cu:180-190, cuda/gemm/fp4_gemm.cu:181-190) for a weight that was quantised once.
 *   w            the packed weight: q [groups * n, k bytes] K-major; scale = float[1] (DSL_W_FP8), 128x128 block
 *                scales [groups, ceil(n/128), k/128] (DSL_W_FP8_BLOCK128) or tiled scale bytes (FP4);
 *                global_scale = device float (NVFP4 only).  DSL_W_BF16: no quantisation, x must be bf16.
 *   group_offsets  int32[groups + 1] device row offsets when w->groups > 1 (ragged expert groups), else ignored
 *   act_scratch  device memory (256-byte aligned) of at least dsl_linear_scratch_bytes(format, M, k, groups) bytes
 *                that receives the quantised activations, their scales and the amax cell; the GEMM of the same
 *                call consumes it, so calls issued in order on one stream may share one area.  Calls that can
 *                overlap on the GPU (different streams) need separate areas, like dsl_epilogue.workspace.
 *   ep           as for dsl_gemm_*; scale_a / scale_b are filled in here (activation scale, weight scale) and
 *                b_is_static is set.  NVFP4 only: a non-NULL ep->scale_a_dev on entry is taken as the activations'
 *                global scale (a calibrated value, device float); the quantiser then needs no amax pass and reads
 *                x once.  Otherwise the global scale is amax(x) / 2688, which costs a pass of its own.
 */
enum { DSL_W_FP8 = 0, DSL_W_FP8_BLOCK128 = 1, DSL_W_NVFP4 = 2, DSL_W_MXFP4 = 3, DSL_W_BF16 = 4 };
typedef struct {
    int format;                 /* DSL_W_* */
    int groups, n, k;           /* weight is [groups, n, k] */
    const void* q;
    const void* scale;
    const float* global_scale;
} dsl_weight;
size_t dsl_linear_scratch_bytes(int format, long long M, int K, int groups);
int dsl_linear(const void* x, int x_dtype, long long M, const dsl_weight* w, const int* group_offsets,
               void* act_scratch, size_t act_scratch_bytes, void* C, long long ldc, const dsl_epilogue* ep,
               uint32_t* status, void* stream);

/*
 * The reference's own FP4 container (its "NVFP4" and "MXFP4" are one format, cuda/gemm/fp4_gemm.cu:30-42):
 * e2m1 nibbles with one fp32 scale per 32 contiguous elements of the FLAT buffer.
 * dsl_quant_fp4_ref32 replaces quantize_fp32_to_nvfp4 (fp4_gemm.cu:50-90) bit for bit (scale = max(amax/6,
 * 1e-12), ties to the lower table index): q_out ceil(n/2) bytes, scales_out ceil(n/32) floats.
 * dsl_gemm_fp4_ref32 replaces fp4_gemm (fp4_gemm.cu:95-146) bit for bit: A packed [M,K] (pairs along K),
 * B packed [K,N] (pairs along N), scale_a [M,K/32], scale_b [K/32,N], C fp32 [M,N].  K % 32 == 0, N % 8 == 0.
 * Runs on the integer dot-product units (fp32 scales per 32 cannot ride in the block-scaled MMA).
 */
int dsl_quant_fp4_ref32(const void* x, int dtype, long long n, uint8_t* q_out, float* scales_out, void* stream);
int dsl_gemm_fp4_ref32(const uint8_t* A, const uint8_t* B, float* C, const float* scale_a, const float* scale_b,
                       int M, int N, int K, void* stream);

/*
 * Mixture-of-experts steps either side of the grouped GEMM (the reference stops at the grouped GEMM itself,
 * cuda/gemm/grouped_gemm.cu:79-104; these have no counterpart there).  All deterministic.
 *   dsl_moe_route     logits [tokens, experts] (f32 / bf16) -> ids [tokens, k] (int32, ties to the lower index) and
 *                     weights [tokens, k] = softmax probabilities of the chosen experts (renorm: divided by their sum)
 *   dsl_moe_plan      ids -> offsets [experts+1] (rows per expert, prefix sums: the group_offsets of the GEMMs),
 *                     tile0 [experts+1] (prefix sums of ceil(rows/128): first scale tile of each expert) and
 *                     dest [tokens*k]: row of entry token*k+slot in the expert-sorted order (stable);
 *                     scratch: dsl_moe_plan_scratch_bytes(entries, experts) bytes
 *   dsl_moe_dispatch_fp4  copies the packed rows and scale bytes of tokens quantised ONCE (q_in [tokens, K/2], sf_in
 *                     token-major scale tiles) to their expert-sorted rows for the experts [first, last): q_out
 *                     [rows, K/2], sf_out in the ragged-group tile layout (zero-filled by the caller)
 *   dsl_moe_dispatch_rows the same mapping for plain rows of row_bytes (% 16 == 0) bytes
 *   dsl_moe_combine   out[t, :] = sum over t's slots with a local expert, in slot order, of weight * y[row, :]
 *
 * Token all-to-all (experts split over several GPUs, every GPU owning a share of the tokens): a routed row crosses
 * the link as one record of dsl_moe_wire_bytes(K, format) bytes - the packed e2m1 bytes, then the row's scale bytes
 * in K order (one 32-bit word per 512-byte scale tile of the row), zero-padded to a multiple of 16.
 *   dsl_moe_pack_wire_fp4    rows quantised once per token (q_in, token-major scale tiles sf_in) -> records in the
 *                     expert-sorted order of dest (wire_out [tokens*k, wire bytes]); contiguous runs of it go to
 *                     the GPUs that own the experts
 *   dsl_moe_unpack_wire_fp4  records as they arrived (record r belongs to this GPU's expert ids[r] and takes row
 *                     dest[r] of its expert-sorted order, both from dsl_moe_plan over the arrived rows) -> packed
 *                     rows q_out [rows, K/2] and scale tiles sf_out in the ragged-group layout (zero-filled by the
 *                     caller), i.e. the A operand of the grouped GEMM
 */
int dsl_moe_route(const void* logits, int dtype, int tokens, int experts, int k, int renorm, int* ids_out,
                  float* weights_out, void* stream);
size_t dsl_moe_plan_scratch_bytes(int entries, int experts);
int dsl_moe_plan(const int* ids, int entries, int experts, int* scratch, int* offsets_out, int* tile0_out,
                 int* dest_out, void* stream);
int dsl_moe_dispatch_fp4(const uint8_t* q_in, const uint8_t* sf_in, const int* ids, const int* dest, const int* offsets,
                         const int* tile0, int tokens, int k, int K, int format, int first_expert, int last_expert,
                         uint8_t* q_out, uint8_t* sf_out, void* stream);
int dsl_moe_dispatch_rows(const void* x, const int* ids, const int* dest, const int* offsets, int tokens, int k,
                          long long row_bytes, int first_expert, int last_expert, void* out, void* stream);
int dsl_moe_combine(const void* y, int y_dtype, const int* ids, const int* dest, const int* offsets, const float* weights,
                    int tokens, int k, int d_model, int first_expert, int last_expert, void* out, int out_dtype,
                    void* stream);
size_t dsl_moe_wire_bytes(int K, int format);
/*
 * Sum of the ranks' partial results over peer memory (expert-parallel layer whose ranks keep their own token rows; no
 * counterpart in the reference).  part_ptrs: HOST array of `world` device pointers, entry s = rank s's partial result
 * [total rows, d_model] (float32 or bfloat16, contiguous, 16-byte aligned), each addressable from this device - this
 * rank's own buffer and its peers' buffers mapped by the caller (CUDA IPC / symmetric memory).  Writes
 * out[r, :] = sum over s = 0 .. world-1, in that order, in fp32, of part_s[row0 + r, :] for r < rows.  The peers'
 * buffers are only read, with plain loads (no TMA, no multicast).  The caller orders the call after every rank has
 * finished writing its buffer (a collective or barrier on the stream) and does not overwrite a buffer before every rank
 * has read it (two alternating buffers and one barrier per step suffice).  d_model must be a whole number of 16-byte
 * vectors; at most DSL_MAX_PEERS ranks.
 */
#define DSL_MAX_PEERS 16
int dsl_moe_reduce_pull(const void* const* part_ptrs, int world, long long row0, long long rows, int d_model, int in_dtype,
                        void* out, int out_dtype, void* stream);
int dsl_moe_pack_wire_fp4(const uint8_t* q_in, const uint8_t* sf_in, const int* dest, int tokens, int k, int K, int format,
                          uint8_t* wire_out, void* stream);
int dsl_moe_unpack_wire_fp4(const uint8_t* wire_in, const int* ids, const int* dest, const int* offsets, const int* tile0,
                            int rows, int K, int format, uint8_t* q_out, uint8_t* sf_out, void* stream);

/*
 * dsl_gemm_fp4 for callers that cannot allocate device memory (no counterpart in the
 * reference).  Same operands and result as dsl_gemm_fp4 on a dense problem, but the scratch for
 * partial sums along K is a fixed DSL_STATIC_SCRATCH_BYTES array inside the library instead of
 * ep->workspace (which is ignored), so nothing but inputs and outputs is passed and the call
 * performs no allocation.  Meant for decode-sized problems: it returns DSL_ERR_TOO_LARGE when
 * dsl_workspace_bytes() for the problem exceeds the array (e.g. 32 tokens against more than
 * 126 x 128 columns on a 148-SM part); problems that need no scratch at all pass through.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress);
 * make that call before any stream capture.  All calls share the one array and it keeps the
 * previous call's contents.  Partial sums are always written by a call before that call reads
 * them.  The arrival words in the array's first 64 KiB are the exception: they are read first,
 * and are safe because the array starts zeroed, nothing but those words is ever stored there,
 * each launch tags its words with an epoch of its own and the kernel zeroes a word once its
 * tile is finished.  So nothing needs clearing between calls, but two calls that overlap on
 * the GPU (different streams) race on the array.
 */
#define DSL_STATIC_SCRATCH_BYTES (4u << 20)
int dsl_gemm_fp4_static_scratch(const uint8_t* A, const uint8_t* B, const uint8_t* sfa, const uint8_t* sfb,
                                int format, void* C, long long ldc, long long M, int N, int K,
                                const dsl_epilogue* ep, uint32_t* status, void* stream);

/* Test hook for the entry point above: copies `bytes` bytes between the static array (from `offset`) and the
 * device buffer `user`, into the array when to_array != 0, ordered on `stream`.  Lets a test put foreign
 * bytes into the array before a call and see afterwards what the call wrote.  Not for production use. */
int dsl_selftest_static_scratch_copy(void* user, size_t offset, size_t bytes, int to_array, void* stream);

/* Runs one bounded wait on a barrier nothing ever signals and reports DSL_ST_TIMEOUT_TEST
 * in *status after about `limit_us` microseconds: exercises the give-up path without
 * faulting or hanging the device. */
int dsl_selftest_bounded_wait(uint32_t* status, unsigned limit_us, void* stream);

/* The work list of the group-scaled FP8 CTA-pair kernel for a problem, computed on the HOST by the kernel's own
 * scheduler code (no CUDA call, no GPU needed): for tests that every output element is covered exactly once.
 * group_offsets: HOST int32 [num_groups + 1] row offsets, or NULL for one dense group of m_total rows; they pass through
 * the kernel's own sanitiser (entries clamped to [0, m_total] and raised to their predecessor), so malformed offsets
 * are accepted here and the items show what the kernel would do with them.  pairs = CTA
 * pairs of the launch (74 on a 148-SM part), band <= 0 = the default raster band, whole_tiles_only = 1 switches the
 * cutting of the last round off.  Item i (it runs on pair i % pairs, in order) is written to out[6 i ..] as
 * {pair, group, row0, row_end, n0, width}: rows [row0, min(row0 + 256, row_end)) x columns [n0, min(n0 + width, N)).
 * Returns the number of items, DSL_ERR_TOO_LARGE when it exceeds max_items, or another DSL_ERR_*. */
int dsl_selftest_groupwise_schedule(const int32_t* group_offsets, int num_groups, long long m_total, int N, int pairs,
                                    int band, int whole_tiles_only, int32_t* out, int max_items);

#ifdef __cplusplus
}
#endif
#endif /* DSLGEMM_H_ */
