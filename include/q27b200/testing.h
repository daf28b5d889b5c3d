/* C ABI of libq27b200_test.so: scaffolding for the test suite, kept OUT of the product library libq27b200.so.
 *   - host-only views of the work split (no CUDA call), so the CPU tests can check coverage and order;
 *   - a deliberately naive device GEMM as an independent cross-check;
 *   - a self-test that drives the C++ launchers of include/q27b200/kernels.h (the face the engine links against)
 *     from C++, including their exception on a failed precondition.
 * Same conventions as capi.h: 0 on success, -1 on failure with q27_last_error() set. Nothing here has a
 * counterpart in the reference; no product code path calls into this library.
 */
#ifndef Q27B200_TESTING_H_
#define Q27B200_TESTING_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Work split of one weight-streaming GEMM for `slots` CTAs that can run at once (the launchers use two per
 * multiprocessor): the pieces {tile, c0, c1, slot} of CTA `cta` (at most `cap`); returns their number.
 * split_out: 0 = contiguous unit ranges, s >= 1 = s aligned K-parts per tile. */
int q27b_skinny_plan(int N, int K, int slots, int cta, int* seg, int cap, int* grid_out, int64_t* units_out,
                     int* split_out);
/* The partial-tile slots a tile is summed from, in summation order; returns their number (1 = not cut). */
int q27b_skinny_tile_parts(int N, int K, int slots, int tile, int* slot, int cap);
/* Schedule of a grouped launch over n problems of shapes (N[i], K[i]) for `slots` resident CTAs: writes up to `cap`
 * pieces as 9 ints each {cta, problem, tile, c0, c1, slot, nparts, slot0, sums}, grouped by CTA in the order the CTA
 * walks them (whole_tiles != 0: no tile is cut, see Q27B_GROUP_WHOLE_TILES, 2: tiles of 256 weight rows as planned for 33..128 tokens; problem order, the launcher's; rotate != 0: every CTA starts at a different point of its list, kept for
 * experiments); sums = 1 marks the one piece of a cut tile whose CTA sums the tile; returns the number of pieces. ctas_out / slots_out / counters_out: CTAs launched, partial-tile slots and arrival
 * counters of the workspace. */
int q27b_skinny_group_plan(int n, const int* N, const int* K, int slots, int whole_tiles, int rotate, int* pieces, int cap, int* ctas_out,
                           int64_t* slots_out, int* counters_out);

/* d[M][N] = alpha * A . B^T, one thread per output, fp32 accumulation in ascending K order. Synchronous. */
int q27t_ref_gemm_fp4(int M, int N, int K, const uint8_t* a, const uint8_t* a_sf, const uint8_t* b, const uint8_t* b_sf,
                      float alpha, float* d);

/* Drives q27::quant_fp4 -> q27::skinny_fp4 (with `nseg` AlphaSegments) on x fp32 [M][K] into d [M][N], and
 * q27::gemm_fp4_glu on the quantised x against gate_up [2 I][K] into (h_q, h_sf), all through the C++ launchers on
 * a stream of its own, then synchronises. Every pointer is a device pointer except seg_begin / seg_alpha. */
int q27t_cxx_launchers(const float* x, int M, int K, float in_scale, uint8_t* q, uint8_t* sf, int N, const uint8_t* w,
                       const uint8_t* w_sf, int nseg, const int* seg_begin, const float* seg_alpha, float* d, void* ws,
                       size_t ws_bytes, int I, const uint8_t* gate_up, const uint8_t* gate_up_sf, float alpha_gate,
                       float alpha_up, float out_scale, uint8_t* h_q, uint8_t* h_sf);
/* Calls q27::skinny_fp4 with M = 0 and q27::quant_fp4 with K = 8: returns 1 when both throw std::runtime_error whose
 * message starts with "check failed", 0 otherwise. No kernel is launched. */
int q27t_cxx_throws(void);

#ifdef __cplusplus
}
#endif
#endif /* Q27B200_TESTING_H_ */
