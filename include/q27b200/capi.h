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

/* ---- activation quantisers (K, I multiples of 64; x 16-byte aligned) ------------------------------------------ */

/* fp32 [M][K] -> codes [M][K/2] + swizzled scales. Replaces quant_fp4 (engine/src/kernels.h:124-126,
 * engine/src/kernels.cu:99-113,151-159,663-668). Bit-exact with reference/qwen27b/quant.py:58-67. */
int q27b_quant_fp4(const float* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, void* stream);
/* The same for bf16 input (bf16 -> fp32 is exact, so the result equals quantising the widened values). New entry
 * point (the benchmark's activations are bf16); the reference quantises bf16 only inside silu_mul_quant_fp4. */
int q27b_quant_fp4_bf16(const void* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf, void* stream);
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
 * address up and clears its counters (a synchronous memset), so make that first call before any stream capture.
 * All calls share the one array and it keeps what the last call left: the kernels leave its counters at zero, the
 * rest needs no clearing; two calls whose kernels overlap on the GPU (different streams) race on it — keep them
 * in stream order. Results are bit-identical to q27b_skinny_fp4. It has no counterpart in the reference, whose
 * callers always pass a workspace (engine/src/kernels.h:240-245). */
int q27b_skinny_fp4_static(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                           const uint8_t* w_sf, int alpha_count, const int* alpha_begin, const float* alpha,
                           const float* c, float beta, float* d, void* stream);
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
/* One thread per output, fp32 accumulation in K order: a slow device-side cross-check for the tests only; no
 * product entry point routes through it. No counterpart in the reference. */
int q27b_ref_gemm_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
                      float alpha, float* d, void* stream);
/* Host-only view of the weight-streaming work split (no CUDA call) for `slots` CTAs that can run at once (the
 * launchers use two per multiprocessor up to M = 64, one above): the pieces {tile, c0, c1, slot} of CTA `cta`;
 * returns the number of pieces. split_out: 0 = contiguous unit ranges, s >= 1 = s aligned K-parts per tile. */
int q27b_skinny_plan(int N, int K, int slots, int cta, int* seg, int cap, int* grid_out, int64_t* units_out,
                     int* split_out);
/* The partial-tile slots a tile is summed from, in summation order; returns their number (1 = the tile is not cut). */
int q27b_skinny_tile_parts(int N, int K, int slots, int tile, int* slot, int cap);

/* ---- synchronous test layer (replaces the q27t_* wrappers, engine/src/capi.cc:498-636) ---------------------------- */

float q27t_last_us(void); /* per-launch time of the last Q27T_REPEAT graph replay (capi.cc:38,57-92) */
int64_t q27t_sf_bytes(int64_t rows, int64_t kblocks);                                  /* capi.cc:565 */
int q27t_quant_fp4(const float* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf); /* capi.cc:498-500 */
int q27t_quant_fp4_bf16(const void* x, int M, int K, float input_scale, uint8_t* q, uint8_t* sf);
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
int q27t_ref_gemm_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
                      float alpha, float* d);
int q27t_skinny_fp4_static(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                           const uint8_t* w_sf, float alpha, const float* c, float beta, float* d);
/* Average microseconds of `iters` GEMMs cycling through `nbuf` weight copies (w_stride / sf_stride bytes apart) so
 * that weights never come from L2; `us` is a HOST pointer. Replaces q27t_bench_gemm (capi.cc:607-636). */
int q27t_bench_gemm(int many, int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* w,
                    const uint8_t* w_sf, int64_t w_stride, int64_t sf_stride, int nbuf, int iters, float* d, void* ws,
                    size_t ws_bytes, float* us);

#ifdef __cplusplus
}
#endif
#endif /* Q27B200_CAPI_H_ */
