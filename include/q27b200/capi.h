/* C ABI of libq27b200.so: the NVFP4 activation quantisers and the NVFP4 x NVFP4 GEMMs for sm_100a.
 *
 * Conventions (those of the reference's C layer, engine/src/capi.cc:19-36,157-158):
 *   - every function returns 0 on success and -1 on failure; q27_last_error() then holds a thread-local message;
 *   - all pointers are DEVICE pointers unless said otherwise; the caller owns every buffer; nothing here
 *     allocates, frees or synchronises unless said otherwise;
 *   - q27b_* functions enqueue work on `stream` (a cudaStream_t passed as void*) and return at once; they may be
 *     captured into a CUDA graph after one eager call per kernel variant and device (the first call of a
 *     variant sets a function attribute);
 *   - q27t_* functions are the synchronous one-kernel wrappers the tests and the benchmark use: they synchronise
 *     the device, run on a private stream, synchronise again and fail if a kernel reported a timed-out wait.
 *
 * Programmatic dependent launch. Every kernel here is launched with the programmatic-stream-serialization
 * attribute (unless Q27_NO_PDL=1 is in the environment at launch time): it may START while the kernel before it in
 * the stream is still running. What a kernel reads before its griddepcontrol.wait is only what callers promise is
 * immutable by then: the GEMMs fetch their first WEIGHT tiles and weight scales (and the grouped GEMM its table)
 * that early. The contract, which the engine's "weights are immutable after load" satisfies by itself: w and w_sf
 * of a GEMM must not be written by the kernel that immediately precedes the GEMM in its stream. Anything earlier is
 * safe, because every kernel of this library releases its successor only after its own wait on its predecessor has
 * returned. A caller that does produce weights with the directly preceding kernel (a device-side weight update, a
 * quantiser making the B operand) sets Q27_NO_PDL=1 for that launch or puts any other kernel in between.
 * Activations, residuals and outputs are touched only after the wait and carry no such condition.
 *
 * Timed-out waits. Every wait inside a kernel is bounded; when one runs out the kernel records a code that
 * q27b_device_status returns, and ends. Such a kernel may have left arrival counters non-zero and partial tiles
 * unpublished: before the next call that uses the same workspace, the caller must zero its first 16 KiB again
 * (q27b_skinny_fp4_static does this for the library's own scratch by itself).
 *
 * Operand formats: E2M1 codes two per byte (low nibble = even K index), one E4M3 scale per 16 K-elements stored in
 * 512-byte atoms of 128 rows x 4 k-blocks (q27b_sf_offset), an fp32 tensor scale folded into `alpha` by the
 * caller. Rows of a scale buffer past the last real row are never read as valid.
 *
 * "Replaces" names the reference interface each entry point stands in for (paths inside the reference project).
 */
#ifndef Q27B200_CAPI_H_
#define Q27B200_CAPI_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Message of the last failed call on this thread. Replaces q27_last_error (engine/src/capi.cc:157). */
const char* q27_last_error(void);

/* ---- layouts ------------------------------------------------------------------------------------------------ */

/* Bytes of a swizzled scale buffer for [rows][kblocks]. Replaces sf_bytes (engine/src/kernels.h:197-199). */
int64_t q27b_sf_bytes(int64_t rows, int64_t kblocks);
/* Byte offset of scale (row, kb). Replaces sf_offset (engine/src/kernels.h:192-195). */
int64_t q27b_sf_offset(int64_t row, int64_t kb, int64_t kblocks);
/* Row of gate (half 0) / up (half 1) row r in the interleaved gate | up. Replaces glu_row (kernels.h:186). */
int64_t q27b_glu_row(int64_t r, int half);
/* Row-major scales [rows][kblocks] -> swizzled layout; glu_half 0 / 1 places the rows of the gate / the up into
 * the interleaved matrix starting at dst, -1 keeps the row order. Replaces swizzle_sf (engine/src/kernels.h:191,
 * engine/src/kernels.cu:587-592,824-827). */
int q27b_swizzle_sf(const uint8_t* src, int rows, int kblocks, uint8_t* dst, int glu_half, void* stream);

/* ---- checkpoints (load time; csrc/checkpoint.cu) -------------------------------------------------------------- */

/* Bytes [off, off + len) of the gate (half 0) or the up (half 1) matrix, in HOST memory at host_src, copied to their
 * places in the interleaved gate | up that starts at dst (device): blocks of `block` bytes (64 rows), the gate's block b
 * at 2 b, the up's at 2 b + 1; whole blocks go as one strided copy. Asynchronous on `stream`; host_src must stay
 * untouched until the copy has run. Replaces copy_glu (engine/src/weights.cc:218-234). */
int q27b_copy_glu(void* dst, size_t off, const void* host_src, size_t len, size_t block, int half, void* stream);

/* A safetensors checkpoint: one file, or a directory whose *.safetensors files are its shards. Replaces the reading
 * side of SafeTensors (engine/src/safetensors.h:24-41: has / info / read_range). */
typedef struct q27b_ckpt q27b_ckpt;
int q27b_ckpt_open(const char* path, q27b_ckpt** out);
void q27b_ckpt_close(q27b_ckpt* c);
int q27b_ckpt_count(const q27b_ckpt* c); /* tensors in the checkpoint */
/* 0 and the tensor's dtype ("U8", "F8_E4M3", "F32", "BF16", ...), shape and size; 1 if the checkpoint has no such
 * tensor (not an error); -1 on bad arguments. Any output pointer may be null. */
int q27b_ckpt_tensor(const q27b_ckpt* c, const char* name, char* dtype, int dtype_cap, int64_t* shape, int shape_cap, int* ndim,
                     int64_t* nbytes);
/* Bytes [begin, begin + len) of a tensor into host memory. */
int q27b_ckpt_read(const q27b_ckpt* c, const char* name, int64_t begin, int64_t len, void* host_dst);

/* One NVFP4 projection as the checkpoint stores it, in either naming (modelopt: <p>.weight, .weight_scale,
 * .weight_scale_2, .input_scale; compressed-tensors: <p>.weight_packed, .weight_scale, .weight_global_scale =
 * 1 / weight_scale_2, .input_global_scale = 1 / input_scale). The LinearFp4 record of the reference
 * (engine/src/weights.h:25-31) as filled by Weights::fp4 (engine/src/weights.cc:125-141). */
typedef struct q27b_fp4_layer {
  int out, in;              /* rows of the weight, reduction length */
  float w_scale2, in_scale; /* tensor scales of the weight and of its activation; alpha = in_scale * w_scale2 */
  int compressed_tensors;   /* 1: the reciprocal-scale naming */
} q27b_fp4_layer;
int q27b_ckpt_fp4_layer(const q27b_ckpt* c, const char* prefix, q27b_fp4_layer* info);
/* Uploads the projection into the layout the GEMMs read: codes to w (device, [out][in / 2]), block scales swizzled
 * to sf (device, q27b_sf_bytes(out, in / 16) bytes of a buffer the caller zeroed; for gate | up the buffer of the
 * whole interleaved matrix). glu_half -1: as stored; 0 / 1: this projection is the gate / the up of an MLP and w, sf
 * are the START of the interleaved gate | up matrix (out must be a multiple of 64). scratch: device memory of at
 * least out * in / 16 bytes (the row-major scales on their way). Reads through two pinned staging buffers owned by the
 * handle; returns after the stream has been synchronised. Load-time only. */
int q27b_ckpt_load_fp4(q27b_ckpt* c, const char* prefix, int glu_half, uint8_t* w, uint8_t* sf, void* scratch, size_t scratch_bytes,
                       void* stream);

/* ---- activation quantisers (K, I multiples of 64; x 16-byte aligned) ------------------------------------------ */

/* fp32 [M][K] -> codes [M][K/2] + swizzled scales. Replaces quant_fp4 (engine/src/kernels.h:124-126,
 * engine/src/kernels.cu:99-113,151-159,663-668). Bit-exact with reference/qwen27b/quant.py:58-67. */
int q27b_quant_fp4(const float* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, void* stream);
/* The same for bf16 input (bf16 -> fp32 is exact, so the result equals quantising the widened values). New entry
 * point (the benchmark's activations are bf16); the reference quantises bf16 only inside silu_mul_quant_fp4. */
int q27b_quant_fp4_bf16(const void* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, void* stream);
/* Several activations quantised by ONE launch (a decode layer quantises three small activations, and a launch
 * costs more than the work). jobs_host: HOST array of n jobs, read for validation and for the grid size; jobs_dev:
 * the same array in device memory, read by the kernel, or NULL for n <= 4 (the jobs then travel in the launch
 * parameters). No counterpart in the reference, which fuses its quantisers into the producing kernels instead. */
typedef struct q27b_quant_job {
  const void* x;     /* fp32 or bf16 [M][K], 16-byte aligned */
  uint8_t* q;        /* codes [M][K/2], 8-byte aligned */
  uint8_t* sf;       /* swizzled scales, 4-byte aligned */
  int M, K;          /* K a multiple of 64 */
  float input_scale;
  int bf16;          /* non-zero: x is bf16 */
} q27b_quant_job;
int q27b_quant_fp4_batch(const q27b_quant_job* jobs_host, const q27b_quant_job* jobs_dev, int n, void* stream);
/* RMSNorm over D (a multiple of 512, at most 16384) with zero-centred weights, x / rms(x) * (1 + w), per token, fused
 * with the quantiser: writes the fp32 result to out (may be null) and, when q is not null, its NVFP4 quantisation
 * (exactly quant_fp4 of the fp32 result). cap (optional): a bf16 copy of the input rows, cap_ld elements apart;
 * rstd (optional): 1 / rms per token. Replaces rmsnorm_quant for QuantOut::kFp4 / kNone (engine/src/kernels.h:131-136,
 * engine/src/kernels.cu:211-262,718-726); the FP8 kinds are not part of this path. */
int q27b_rmsnorm_quant_fp4(const float* x, const void* w_bf16, int T, int D, float eps, float* out, float input_scale,
                           uint8_t* q, uint8_t* sf, void* cap_bf16, int cap_ld, float* rstd, void* stream);
/* Dynamic per-token quantisation: as quant_fp4 with each row's own tensor scale ascale[m] = amax(row) / (6 * 448)
 * (1 for an all-zero row), which the call writes. The rule of the reference's draft model (engine/src/draft.cu:70-111,
 * where it is fused into the producing kernels); feeds q27b_skinny_fp4_scaled. */
int q27b_quant_fp4_dynamic(const float* x, int M, int K, uint8_t* q, uint8_t* sf, float* ascale, void* stream);
int q27b_quant_fp4_dynamic_bf16(const void* x, int M, int K, uint8_t* q, uint8_t* sf, float* ascale, void* stream);
/* Load-time weight quantiser: bf16 W[M][K] -> codes q[M][K/2] and swizzled scales, value = global * scale * e2m1,
 * each block's scale code searched (4 codes below to 8 above the code of amax / 6) for the smallest squared error.
 * Replaces quant_fp4_weight (engine/src/kernels.h:130, engine/src/kernels.cu:167-206,670-674). */
int q27b_quant_fp4_weight(const void* w, int M, int K, float global, uint8_t* q, uint8_t* sf, void* stream);
/* silu(gate) * up, then quantised; gate / up rows ld elements apart. Replaces silu_mul_quant_fp4
 * (engine/src/kernels.h:137-141, engine/src/kernels.cu:319-339,728-743). */
int q27b_silu_mul_quant_fp4(const float* gate, const float* up, int64_t ld, int T, int I, float input_scale,
                            uint8_t* q, uint8_t* sf, void* stream);
int q27b_silu_mul_quant_fp4_bf16(const void* gate, const void* up, int64_t ld, int T, int I, float input_scale,
                                 uint8_t* q, uint8_t* sf, void* stream);
/* The same from the [T][2 I] output of the interleaved gate | up weights, applying the two alphas here. Replaces
 * silu_mul_quant_fp4_glu (engine/src/kernels.h:142-147, engine/src/kernels.cu:745-759). */
int q27b_silu_mul_quant_fp4_glu(const float* gu, int T, int I, float alpha_gate, float alpha_up, float input_scale,
                                uint8_t* q, uint8_t* sf, void* stream);
int q27b_silu_mul_quant_fp4_glu_bf16(const void* gu, int T, int I, float alpha_gate, float alpha_up,
                                     float input_scale, uint8_t* q, uint8_t* sf, void* stream);

/* ---- weight-streaming GEMM, 1 <= M <= 128 (N multiple of 128, K multiple of 64) -------------------------------- */

/* D[M][N] = alpha(n) * A . W^T (+ beta * C), fp32. alpha[i] applies from column alpha_begin[i] on (1..4
 * segments, HOST arrays). c may alias d or be null. ws: at least q27b_skinny_workspace_bytes(M, N, K) bytes,
 * 16-byte aligned, shared by all calls of a stream in stream order; it must be zeroed once before the first call
 * (its first 16 KiB hold per-tile arrival counters, which every call leaves at zero, exactly the reference's
 * contract, engine/src/kernels.h:240-242). A token's result is bit-identical whatever M (1..128) it is computed
 * with. Replaces skinny_fp4
 * (engine/src/kernels.h:240-245, engine/src/skinny.cu:462-549; the reference stops at M = 64). */
int q27b_skinny_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w, const uint8_t* w_sf,
                    int alpha_count, const int* alpha_begin, const float* alpha, const float* c, float beta, float* d,
                    void* ws, size_t ws_bytes, void* stream);
/* The same with bf16 output (the fp32 result rounded to nearest even), no residual. New entry point. */
int q27b_skinny_fp4_bf16(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                         const uint8_t* w_sf, int alpha_count, const int* alpha_begin, const float* alpha, void* d,
                         void* ws, size_t ws_bytes, void* stream);
/* gate | up on the interleaved [2 I][K] weights with the epilogue d[M][I] = bf16(silu(alpha_gate * gate) *
 * (alpha_up * up)). New entry point; composes skinny_fp4 with silu_mul of the reference
 * (engine/src/model.cc:1054-1096, reference/qwen27b/model.py:182-185). */
int q27b_skinny_fp4_glu_bf16(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                             const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, void* d, void* ws,
                             size_t ws_bytes, void* stream);
/* q27b_skinny_fp4 for callers that cannot provide a workspace because they may not allocate device memory (a
 * process whose memory plan is frozen, a plug-in loaded into one): the scratch is a
 * fixed array inside the library image, 7.8 MiB per GPU that loads the library, held until the process exits.
 * Limit: 1 <= M <= 16 (decode / speculative-verify batches); a larger M is rejected with a message. Nothing is
 * allocated or freed, here or in anything this calls. The FIRST call on each device looks the array's device
 * address up and clears its counters (a memset enqueued on `stream` ahead of the kernel), so make that first call
 * before any stream capture. The counters are cleared the same way again on the first call after
 * q27b_device_status has reported a timed-out wait.
 * All calls share the one array and it keeps what the last call left: the kernels leave its counters at zero, the
 * rest needs no clearing; two calls whose kernels overlap on the GPU (different streams) race on it — keep them
 * in stream order. Results are bit-identical to q27b_skinny_fp4. It has no counterpart in the reference, whose
 * callers always pass a workspace (engine/src/kernels.h:240-245). */
int q27b_skinny_fp4_static(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                           const uint8_t* w_sf, int alpha_count, const int* alpha_begin, const float* alpha,
                           const float* c, float beta, float* d, void* stream);
/* ---- grouped weight-streaming GEMM: a list of skinny GEMMs in ONE persistent launch ---------------------------------
 *
 * No counterpart in the reference, which launches one kernel per projection and hides the launch boundaries with
 * CUDA graphs and programmatic dependent launch (engine/src/launch.cuh:1-8, engine/src/skinny.cu:225-237). On this
 * GPU a decode GEMM needs 2-4 us of HBM time and a launch boundary costs more than that, so here every CTA streams
 * its share of the weight tiles of ALL problems of the group back to back. By default each problem keeps the K split
 * of its stand-alone launch: the results are bit-identical to q27b_skinny_fp4 / _bf16 / _glu_bf16 called one by one.
 *
 * One problem of a group; all pointers are device pointers, all problems share the token count M of the group. */
typedef struct q27b_group_problem {
  int N;              /* weight rows (2 I for the gate | up epilogue), multiple of 128 */
  int K;              /* multiple of 64 */
  int epilogue;       /* 0: fp32 d[M][N] = alpha(n) acc + beta c;  1: bf16 d[M][N] = alpha(n) acc;
                         2: interleaved gate | up weights, bf16 d[M][N/2] = silu(alpha[0] gate) * (alpha_up up) */
  int alpha_count;    /* 1..4 segments of output channels with their own alpha (AlphaSegments) */
  int alpha_begin[4];
  float alpha[4];
  float alpha_up;
  float beta;
  const uint8_t* a;    /* activation codes [M][K/2] */
  const uint8_t* a_sf; /* its swizzled scales */
  const uint8_t* w;    /* weight codes [N][K/2] */
  const uint8_t* w_sf; /* its swizzled scales */
  const float* c;      /* residual [M][N] (fp32 epilogue only; may alias d) or null */
  void* d;             /* output */
} q27b_group_problem;
/* flags of q27b_skinny_group_build. WHOLE_TILES: no tile is cut along K. A group with many tiles (several layers) fills
 * the GPU evenly without the K split, writes no partial tiles and sums nothing - the fastest form at every M. Every
 * output is then one accumulation chain over all of K, so the results are bit-identical to the many-row GEMM
 * (q27b_gemm_fp4 / _bf16 / _glu_bf16) rather than to the weight-streaming launch. With few tiles (one layer) the
 * CTAs are loaded unevenly; the table's header reports the imbalance, and the default mode is the better choice. */
#define Q27B_GROUP_WHOLE_TILES 1
/* With WHOLE_TILES, 33..128 tokens and every weight a multiple of 256 rows the group is planned on tiles of
 * 256 weight rows with the tokens on the MMA's M side (fewer activation bytes into the SM per weight byte). TOKENS_ON_N
 * keeps the few-token roles instead; the fused gather (q27b_skinny_fp4_group_gather) needs it. Same bits either way. */
#define Q27B_GROUP_TOKENS_ON_N 2
/* Plans the group for 1 <= M <= 128 on the current device and writes its table: tensor maps of every operand, and
 * for every CTA the pieces {problem, weight tile, K range} it streams, longest piece first onto the least loaded
 * CTA, walked in problem order. HOST function, called once per (problem list, M): `problems` and `table_host` are
 * HOST memory. With table_host == NULL it only reports sizes. The caller copies the table_bytes bytes of
 * table_host to 128-byte aligned device memory (a plain cudaMemcpy) and keeps both copies for the launches. ws_bytes:
 * the workspace the launches need, zeroed once by the caller (arrival counters at its head, which every launch
 * leaves at zero; after a launch that reported a timed-out wait, zero it again). */
int q27b_skinny_group_build(int M, int n_problems, const q27b_group_problem* problems, int flags, void* table_host,
                            size_t table_cap, size_t* table_bytes, size_t* ws_bytes);
/* Enqueues the group on `stream`: one launch, nothing allocated or copied (capturable after one eager call per
 * token-tile size and device). Operands, weights and the table must be complete before the kernel that precedes
 * this one in the stream STARTS (see "programmatic dependent launch" above), except the activations, which may be
 * written by the preceding kernel. Launches sharing a workspace must not overlap on the GPU. */
int q27b_skinny_fp4_group(const void* table_host, const void* table_dev, void* ws, size_t ws_bytes, void* stream);

/* ---- the gather fused into the grouped launch (several GPUs, weights sharded along N) -----------------------------
 *
 * Every GPU computes its block of output columns and all GPUs need all blocks. Instead of a collective after the
 * kernel, the epilogue stores every output twice over: into this GPU's memory and, through peer-mapped pointers, into
 * every peer's (plain stores; no multicast, no load from a peer), so the transfer over NVLink overlaps the weight
 * stream. All outputs of the group must lie in ONE region of this GPU's memory; the copy of local address x in peer j
 * is x + out_delta[j]. Each GPU owns a signal block of 16 int32 words in peer-accessible memory, zeroed once: the last
 * CTA of a launch raises word `my_slot` in every peer's block; q27b_group_gather_wait, enqueued behind the launch,
 * returns on the device once every listed peer has raised its word for this step (a bounded wait: status 8 if a peer
 * never reports). The steps of all GPUs must be issued in the same order. No counterpart in the reference (one GPU). */
typedef struct q27b_group_peers {
  int n_peers;               /* 1..7 */
  int my_slot;               /* 0..7: this GPU's word in every signal block (its rank) */
  int64_t out_delta[7];      /* multiples of 16 */
  int32_t* signals;          /* this GPU's signal block */
  int32_t* peer_signals[7];  /* the peers' signal blocks (peer-mapped device pointers) */
} q27b_group_peers;
int q27b_skinny_fp4_group_gather(const void* table_host, const void* table_dev, void* ws, size_t ws_bytes,
                                 const q27b_group_peers* peers, void* stream);
/* peer_slots: the n_peers slots (0..7) to wait for; HOST array. */
int q27b_group_gather_wait(int32_t* signals, int n_peers, const int* peer_slots, void* stream);
/* The same for the prefill gate | up GEMM (q27b_gemm_fp4_glu_bf16 on CTA pairs: M > 128, 2 I a multiple of 256): its
 * epilogue stores every 32-byte piece of the bf16 output into the peers' copies as well, the last CTA raises the
 * signal, q27b_group_gather_wait waits for the peers. d must lie in the peer-mirrored region. At 8 GPUs the floor of
 * this step is the transfer itself (7/8 of the 142.6 MB output into every GPU: 162 us at the 770 GB/s a peer copy
 * reaches here), against about 50 us of GEMM per GPU. */
int q27b_gemm_fp4_glu_bf16_gather(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                                  const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, void* d,
                                  const q27b_group_peers* peers, void* stream);

/* d[m][n] = (A . W^T)[m][n] * (wscale[n] * ascale[m]), fp32: per-output-channel weight scales and per-token
 * activation scales (weights quantised at load, activations quantised dynamically). Replaces skinny_fp4_scaled
 * (engine/src/kernels.h:255-256, engine/src/skinny.cu:402,456,568-572). */
int q27b_skinny_fp4_scaled(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const float* ascale,
                           const uint8_t* w, const uint8_t* w_sf, const float* wscale, float* d, void* ws,
                           size_t ws_bytes, void* stream);
/* Workspace bytes of the calls above on the current device (-1 without a device). The reference sizes its
 * workspace at 32 MiB (engine/src/model.h:462), which covers every shape up to M = 64 on a 148-SM device; the
 * bound is 16 KiB + 4 * SMs * M * 512 bytes (38.8 MiB at M = 128). */
int64_t q27b_skinny_workspace_bytes(int M, int N, int K);

/* ---- many-row GEMM, any M (N and K multiples of 128) ------------------------------------------------------------ */

/* D = alpha * A . B^T + beta * C, fp32; M == 0 is a no-op. Replaces gemm_fp4 (engine/src/kernels.h:203-206,
 * engine/src/gemm_mma.cu:585-621). */
int q27b_gemm_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
                  float alpha, const float* c, float beta, float* d, void* stream);
/* bf16 output = the fp32 result rounded. Replaces gemm_fp4_bf16 (engine/src/kernels.h:207-209,
 * engine/src/gemm_mma.cu:623-626). */
int q27b_gemm_fp4_bf16(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b,
                       const uint8_t* b_sf, float alpha, void* d, void* stream);
/* gate | up GEMM on interleaved weights with d[M][I] = bf16(silu(alpha_gate * gate) * (alpha_up * up)). Stands in
 * for gemm_fp4_glu (engine/src/kernels.h:216-221, engine/src/gemm_mma.cu:350-399,646-652) with the bf16 output the
 * benchmark configurations ask for instead of re-quantised NVFP4. */
int q27b_gemm_fp4_glu_bf16(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                           const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, void* d, void* stream);
/* gate | up GEMM on interleaved weights with silu(alpha_gate * gate) * (alpha_up * up) quantised to NVFP4 in the
 * epilogue: q [M][I / 2] codes and q_sf swizzled scales ([M rows][I / 16 blocks]) are the activation of the down
 * GEMM, quantised with the tensor scale out_scale; gate and up are never rounded to bf16. Replaces gemm_fp4_glu
 * (engine/src/kernels.h:216-221, engine/src/gemm_mma.cu:350-399,646-652). Scale bytes of rows past M inside the
 * last 128-row atom are left untouched. */
int q27b_gemm_fp4_glu(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                      const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, float out_scale, uint8_t* q,
                      uint8_t* q_sf, void* stream);

/* ---- diagnostics -------------------------------------------------------------------------------------------------- */

/* 1 if the optional single-GPU library libq27b200_quad.so (csrc/quad_gemm.cu: the many-row GEMM on clusters of four
 * CTAs that share their weight tile through TMA multicast of this GPU's own memory) lies beside this library and was
 * loaded. With Q27B_MANY=quad (read at every launch, like pairs | wide | narrow) q27b_gemm_fp4 / _bf16 / _glu_bf16 then run
 * it for M > 128 in an even number of 256-token tiles with N and K multiples of 256: same bits as the pair kernel, 29 %
 * fewer bytes out of L2 per flop. It is opt-in because it measured no faster here (the prefill GEMM is bound by the
 * board's power cap). The fused gather never uses it. */
int q27b_quad_available(void);

/* Synchronises the device, returns and clears the status word kernels set when a bounded wait runs out
 * (0 = none; codes in csrc/ptx_sm100.cuh). No counterpart in the reference, whose kernels wait unboundedly. */
int q27b_device_status(uint32_t* status);
/* Self-test of that mechanism: launches one thread that waits, for at most budget_us microseconds (1..100000), on
 * a barrier nothing arrives at; the wait gives up, the kernel ends normally and q27b_device_status then reports 6.
 * Nothing faults or hangs. No counterpart in the reference. */
int q27b_probe_wait_timeout(int budget_us, void* stream);
/* Timeline tracing for performance work: when buf is not null, the GEMM kernels launched afterwards store
 * %globaltimer samples into it, buf[cta][4][64] uint64 (kind 0: load issued, 1: stage ready for the MMAs, 2: stage
 * committed, 3: CTA milestones), zero meaning "not reached"; null switches it off. Host-side setting read at launch
 * time; no counterpart in the reference. */
int q27b_trace_set(void* buf);
/* ---- synchronous test layer (replaces the q27t_* wrappers, engine/src/capi.cc:498-636) ---------------------------- */

float q27t_last_us(void); /* per-launch time of the last Q27T_REPEAT graph replay (capi.cc:38,57-92) */
int64_t q27t_sf_bytes(int64_t rows, int64_t kblocks);                                  /* capi.cc:565 */
int q27t_quant_fp4(const float* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf); /* capi.cc:498-500 */
int q27t_quant_fp4_bf16(const void* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf);
/* hidden size 5120; kind 0: fp32 output only, 2: + NVFP4 (the reference's QuantOut kinds; capi.cc:519-522) */
int q27t_rmsnorm_quant(const float* x, const void* w_bf16, int T, float eps, float* out, int kind, float in_scale,
                       uint8_t* q, uint8_t* sf);
int q27t_quant_fp4_weight(const void* w, int M, int K, float global, uint8_t* q, uint8_t* sf); /* (new wrapper) */
int q27t_quant_fp4_dynamic(const float* x, int M, int K, uint8_t* q, uint8_t* sf, float* ascale); /* (new wrapper) */
int q27t_skinny_fp4_scaled(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const float* ascale,
                           const uint8_t* w, const uint8_t* w_sf, const float* wscale, float* d, void* ws,
                           size_t ws_bytes);                                            /* (new wrapper) */
int q27t_silu_mul_quant_fp4(const float* g, const float* u, int64_t ld, int T, int I, float in_scale, uint8_t* q,
                            uint8_t* sf);                                               /* capi.cc:523-526 */
int q27t_silu_mul_quant_fp4_bf16(const void* g, const void* u, int64_t ld, int T, int I, float in_scale, uint8_t* q,
                                 uint8_t* sf);                                          /* capi.cc:527-530 */
int q27t_silu_mul_quant_fp4_glu(const float* gu, int T, int I, float ag, float au, float in_scale, uint8_t* q,
                                uint8_t* sf);                                           /* capi.cc:531-534 */
int q27t_silu_mul_quant_fp4_glu_bf16(const void* gu, int T, int I, float ag, float au, float in_scale, uint8_t* q,
                                     uint8_t* sf);                                      /* capi.cc:535-538 */
int q27t_swizzle_sf(const uint8_t* src, int rows, int kblocks, uint8_t* dst);            /* capi.cc:559-561 */
int q27t_swizzle_sf_glu(const uint8_t* src, int rows, int kblocks, uint8_t* dst, int half); /* capi.cc:562-564 */
int q27t_gemm_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
                  float alpha, const float* c, float beta, float* d);                   /* capi.cc:566-569 */
int q27t_gemm_fp4_bf16(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b,
                       const uint8_t* b_sf, float alpha, void* d);                      /* capi.cc:539-542 */
int q27t_gemm_fp4_glu_bf16(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                           const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, void* d);
int q27t_gemm_fp4_glu(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                      const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, float out_scale, uint8_t* q,
                      uint8_t* q_sf);                                                  /* capi.cc:570-574 */
int q27t_skinny_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w, const uint8_t* w_sf,
                    float alpha, const float* c, float beta, float* d, void* ws, size_t ws_bytes); /* capi.cc:599-602 */
int q27t_skinny_fp4_segments(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                             const uint8_t* w_sf, int count, const int* begin, const float* alpha, const float* c,
                             float beta, float* d, void* ws, size_t ws_bytes);
int q27t_skinny_fp4_bf16(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                         const uint8_t* w_sf, float alpha, void* d, void* ws, size_t ws_bytes);
int q27t_skinny_fp4_glu_bf16(int M, int I, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* gate_up,
                             const uint8_t* gate_up_sf, float alpha_gate, float alpha_up, void* d, void* ws,
                             size_t ws_bytes);
int q27t_skinny_fp4_static(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                           const uint8_t* w_sf, float alpha, const float* c, float beta, float* d);
int q27t_skinny_fp4_group(const void* table_host, const void* table_dev, void* ws, size_t ws_bytes);
/* Average microseconds of `iters` GEMMs cycling through `nbuf` weight copies (w_stride / sf_stride bytes apart) so
 * that weights never come from L2; `us` is a HOST pointer. Replaces q27t_bench_gemm (capi.cc:607-636). */
int q27t_bench_gemm(int many, int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                    const uint8_t* w_sf, int64_t w_stride, int64_t sf_stride, int nbuf, int iters, float* d, void* ws,
                    size_t ws_bytes, float* us);

#ifdef __cplusplus
}
#endif
#endif /* Q27B200_CAPI_H_ */
