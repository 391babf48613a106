/* weftmoe_b200 — C ABI of the B200 (sm_100a) routed-MoE expert operator.
 *
 * Plain C linkage, plain pointers and sizes, no C++ or torch types.  Every function returns an
 * int status (WM_OK = 0); wm_last_error() returns the calling thread's last message.  Device
 * pointers are CUDA device addresses of the current device; `stream` is a cudaStream_t passed as
 * void*.  The calls replace the native object behind the reference's Python Tensor API
 * (`TensorRuntime.native`, weftmoe/runtime.py:277-464; pybind surface src/python/runtime.cpp:870-953).
 */
#ifndef WEFTMOE_B200_H_
#define WEFTMOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define WM_API __attribute__((visibility("default")))
#else
#define WM_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes.  The numbering follows the spirit of the reference's NotifyErrorCode
 * (include/weftmoe/api/errors.hpp:12-31): contract violations are distinct from runtime failures. */
enum {
  WM_OK = 0,
  WM_ERR_INVALID = 2,      /* argument / shape / alignment contract violated (ValueError)       */
  WM_ERR_CUDA = 3,         /* a CUDA call failed (RuntimeError)                                   */
  WM_ERR_TIMEOUT = 4,      /* a bounded device wait ran out (TransportTimeout in the reference)   */
  WM_ERR_ROUTE = 5,        /* route id outside [-1, experts) (ExpertOutOfRange)                   */
  WM_ERR_CAPACITY = 6,     /* rows or tokens exceed the prepared capacity (CapacityExceeded)      */
  WM_ERR_STATE = 7         /* call not valid in this state (e.g. tape reused, runtime closed)     */
};

WM_API const char* wm_last_error(void);

/* Diagnostic: one grouped GEMM on caller buffers (synchronises `stream`).
 * kind 0: out[rows,n]   = a[rows,k] * b[g][n,k]^T          (FC2 form)
 * kind 1: out[rows,n]   = a[rows,k] * b[g][k,n]            (dU / dX form)
 * kind 2: out[g][m,n]   = sum_r a[r,m] * b[r,n]            (dW form; k_or_m = m)
 * kind 3: out=u[rows,n] = swiglu(a[rows,k] * b[g][2n,k]^T) * row_prob, aux_out = ab[rows,2n] or NULL
 * group_rows_host[g] = rows of expert g (multiples of 128).  Mirrors the role of the reference's
 * diagnostic fp8_gemm binding (src/python/fp8.hpp:61-174). */
WM_API int wm_debug_grouped_gemm(int kind, const void* a, const void* b, void* out, void* aux_out,
                          const float* row_prob, const int* group_rows_host, int groups, int n,
                          int k_or_m, int* status_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WEFTMOE_B200_H_ */
