/*
 * cce_b200_testing — test and measurement hooks of libcce_b200.so.
 *
 * Nothing here belongs to the path the reference's launchers map to (include/cce_b200.h has
 * that); these entry points let the tests drive the tensor-core pipeline in isolation, make a
 * bounded wait run out, and let the benchmark time and count what the product entry points launch.
 * They have no counterpart in the reference.  Conventions as in cce_b200.h.
 */
#ifndef CCE_B200_TESTING_H_
#define CCE_B200_TESTING_H_

#include "cce_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Plain tensor-core GEMM through the same TMA/tcgen05 pipeline, exported so
 * the pipeline can be tested in isolation:  out[M,N] (+)= A * B^T-like product
 * over K.  a_mn / b_mn select the memory order of the operands:
 *   a_mn = 0: A is [M, K] row-major (lda);  a_mn = 1: A is [K, M] row-major.
 *   b_mn = 0: B is [N, K] row-major (ldb);  b_mn = 1: B is [K, N] row-major.
 * out is fp32 (out_dtype = CCE_DT_F32) or the input type; `accumulate` adds to
 * an fp32 out.  kflags (optional, bytes [ceil(M/128)][ceil(K/64)]) marks the
 * 64-wide K blocks that take part for each 128-row block of the output.
 * The first 4 bytes of `status` receive the kernel status word (may be NULL). */
int cce_b200_gemm(const void* A, const void* B, void* out, int64_t M, int64_t N, int64_t K,
                  int64_t lda, int64_t ldb, int64_t ldo, int32_t dtype, int32_t out_dtype,
                  int32_t a_mn, int32_t b_mn, int32_t accumulate, const uint8_t* kflags,
                  int32_t* status, void* stream);

/* Self-test of the bounded wait every pipeline kernel relies on: one warp waits on a barrier at
 * which nobody arrives, gives up after `limit_cycles` SM cycles (1 .. 2e9), writes its code into
 * status[0] (device memory, 4 bytes) and the kernel returns normally.  Afterwards
 * cce_b200_read_status(status, ...) answers CCE_ERR_KERNEL_WAIT.  Touches no TMA, tensor memory or
 * tensor core; the context stays usable. */
int cce_b200_selftest_wait(int64_t limit_cycles, int32_t* status, void* stream);

/* Per-kernel timing of the tensor-core launches, for benchmarks.  While enabled, every launch
 * of the pipeline kernel is bracketed by a CUDA event pair on its stream.  cce_b200_profile_read
 * waits for the recorded launches, writes the summed milliseconds and the launch counts per
 * kernel mode (index 0: forward log-sum-exp, 1: logit-gradient recompute, 2: dE/dC products)
 * into host arrays of 3 entries each, and forgets the records. */
int cce_b200_profile_enable(int on);
/* Tracing of the pipeline's internal waits.  Give a zeroed device array of 24 uint64 (3 kernel
 * modes x 8); until it is reset to NULL every launch of the pipeline kernel adds, into the 8 words
 * of its mode: [0] cycles the TMA producer waited for a free stage, [1] cycles the MMA issuer
 * waited for a filled stage, [2] cycles it waited for a free accumulator, [3] cycles an epilogue
 * warp waited for a finished accumulator, [4] CTA lifetimes, [5] number of CTAs; all summed over
 * CTAs.  The array belongs to the caller and must outlive the launches.  The counters cost the
 * forward kernel several per cent even when unused, so they exist only in a library built with
 * -DCCE_TRACE=1 (python -m cut_cross_entropy._build --trace -> libcce_b200_trace.so, loaded with
 * CCE_B200_LIB); the default build answers CCE_ERR_UNSUPPORTED to a non-NULL array. */
int cce_b200_profile_wait_counters(void* device_counters /* uint64[24] or NULL */);
int cce_b200_profile_read(double* ms /* host [3] */, int64_t* launches /* host [3] */);
/* SM clock the pipeline kernels really ran at.  Give a device array of 12 uint64 (3 kernel modes x
 * 4); until it is reset to NULL, block 0 of every launch writes into the 4 words of its mode:
 * [0] clock64 and [1] globaltimer (ns) at its start, [2], [3] the same at its end.  (cycles / ns)
 * of the last launch of a mode is the SM clock in GHz during that launch, which a 100 ms
 * nvidia-smi sample cannot resolve.  The array belongs to the caller. */
int cce_b200_profile_clock_words(void* device_words /* uint64[12] or NULL */);
/* How much of the logit-gradient matrix the block-list backward recomputes.  Give a device array
 * of 3 int32; until it is reset to NULL every block-list backward writes {tiles (128 rows x 256
 * columns) it recomputes, tiles in all, passes over the tile pool it needs} into it. */
int cce_b200_profile_tile_counts(void* device_counts /* int32[3] or NULL */);

/* Counters since library load (host side): kernels launched by this library. */
int64_t cce_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* CCE_B200_TESTING_H_ */
