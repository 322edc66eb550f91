/* C interface of libmomijo_b200.so for callers that link the kernel library directly (without
 * Python). Every function returns 0 on success, a negative code for a rejected argument and a
 * positive CUDA error code for a failed launch. Pointers are device pointers unless stated
 * otherwise; `stream` is a cudaStream_t passed as void*. */
#ifndef MOMIJO_B200_H_
#define MOMIJO_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

/* Column sums of a row-major bf16 matrix x[M, N] (row stride ldx elements, a multiple of 8):
 * out[n] = sum_m x[m, n], written as bf16 (out_bf16) or fp32 (out_f32, used when out_bf16 is
 * NULL); with accumulate != 0 the sums are added to the existing output. `scratch` must hold
 * mmj_colsum_splits(M) * N floats. */
int mmj_colsum_splits(int M);
int mmj_colsum_bf16(const void* x, long long ldx, void* out_bf16, float* out_f32, float* scratch,
                    int M, int N, int accumulate, void* stream);

/* The same column sum for callers that cannot allocate device memory (inside a no-allocation
 * region of a memory pool, in a serving loop that has given all free memory to its cache, or in a
 * host application that forbids allocation after start-up). This entry point has no counterpart
 * in the reference framework; it exists only in this library.
 *
 * Instead of caller-provided scratch it uses a 4 MiB array compiled into the library, which each
 * GPU that loads the library keeps until the process exits. Limits and rules:
 *   - N <= mmj_colsum_bf16_static_max_n() (16384); larger N is rejected with code -20 and
 *     mmj_colsum_bf16_static_strerror(code) gives the message;
 *   - it never calls cudaMalloc, cudaFree or any other allocating routine;
 *   - the first call on each device looks up the array's device address (a one-time set-up done
 *     with that device current), so make that first call before starting any stream capture;
 *   - all calls on a device share the array and it keeps the previous call's contents; nothing
 *     needs clearing between calls, but calls that overlap on the GPU race with each other, so
 *     keep them on one stream or order them with events. */
int mmj_colsum_bf16_static_max_n(void);
const char* mmj_colsum_bf16_static_strerror(int code);
int mmj_colsum_bf16_static(const void* x, long long ldx, void* out_bf16, float* out_f32, int M,
                           int N, int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOMIJO_B200_H_ */
