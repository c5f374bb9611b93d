// Complex scalars for the first-order policies (complex64 / complex128, interleaved {re, im}
// exactly as torch stores them).  The policies are written against a scalar type S with
// + and *, S(0) / S(1), ld_ro() and the shfl_*_s() warp shuffles; this header gives both reals and
// Cx<R> all of these, plus the
// conjugate cj() that the adjoint applies to coefficients and saved outputs (identity for reals):
// for complex data the adjoint recurrence runs on conj(a) and the coefficient gradient is
// g[t] * conj(y[t-1]) (philtorch/lti/recur.py:31-57 in the reference's autograd Function).
#pragma once
#include <cuda_runtime.h>

namespace ptb {

template <class R>
struct alignas(2 * sizeof(R)) Cx {
  R re, im;
  Cx() = default;
  __host__ __device__ __forceinline__ Cx(R r) : re(r), im(R(0)) {}
  __host__ __device__ __forceinline__ Cx(R r, R i) : re(r), im(i) {}
  __host__ __device__ __forceinline__ Cx& operator+=(const Cx& o) { re += o.re; im += o.im; return *this; }
  __host__ __device__ __forceinline__ Cx& operator*=(const Cx& o) {
    const R r = re * o.re - im * o.im;
    im = re * o.im + im * o.re;
    re = r;
    return *this;
  }
};

template <class R>
__host__ __device__ __forceinline__ Cx<R> operator+(const Cx<R>& a, const Cx<R>& b) {
  return Cx<R>(a.re + b.re, a.im + b.im);
}
template <class R>
__host__ __device__ __forceinline__ Cx<R> operator-(const Cx<R>& a, const Cx<R>& b) {
  return Cx<R>(a.re - b.re, a.im - b.im);
}
template <class R>
__host__ __device__ __forceinline__ Cx<R> operator*(const Cx<R>& a, const Cx<R>& b) {
  return Cx<R>(a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re);
}

__host__ __device__ __forceinline__ float cj(float v) { return v; }
__host__ __device__ __forceinline__ double cj(double v) { return v; }
template <class R>
__host__ __device__ __forceinline__ Cx<R> cj(const Cx<R>& v) { return Cx<R>(v.re, -v.im); }

// read-only load and warp shuffles of one scalar, real or complex
template <class T> __device__ __forceinline__ T ld_ro(const T* p) { return __ldg(p); }
template <class R>
__device__ __forceinline__ Cx<R> ld_ro(const Cx<R>* p) {
  const R* q = reinterpret_cast<const R*>(p);
  return Cx<R>(__ldg(q), __ldg(q + 1));
}
template <class T> __device__ __forceinline__ T shfl_up_s(const T& v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
template <class T> __device__ __forceinline__ T shfl_down_s(const T& v, int d) { return __shfl_down_sync(0xffffffffu, v, d); }
template <class T> __device__ __forceinline__ T shfl_s(const T& v, int src) { return __shfl_sync(0xffffffffu, v, src); }
template <class R>
__device__ __forceinline__ Cx<R> shfl_up_s(const Cx<R>& v, int d) {
  return Cx<R>(__shfl_up_sync(0xffffffffu, v.re, d), __shfl_up_sync(0xffffffffu, v.im, d));
}
template <class R>
__device__ __forceinline__ Cx<R> shfl_down_s(const Cx<R>& v, int d) {
  return Cx<R>(__shfl_down_sync(0xffffffffu, v.re, d), __shfl_down_sync(0xffffffffu, v.im, d));
}
template <class R>
__device__ __forceinline__ Cx<R> shfl_s(const Cx<R>& v, int src) {
  return Cx<R>(__shfl_sync(0xffffffffu, v.re, src), __shfl_sync(0xffffffffu, v.im, src));
}

}  // namespace ptb
