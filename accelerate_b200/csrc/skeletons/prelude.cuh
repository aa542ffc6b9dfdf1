// Common prelude of every generated kernel source (compiled by NVRTC for
// sm_100a with --fmad=false, no fast-math).  Scalar helpers reproduce the
// primitive semantics of the reference interpreter (Interpreter.hs:1154-1416).

typedef signed char i8;
typedef short i16;
typedef int i32;
typedef long long i64;
typedef unsigned char u8;
typedef unsigned short u16;
typedef unsigned int u32;
typedef unsigned long long u64;
typedef float f32;
typedef double f64;

#define ACC_FULL_MASK 0xffffffffu
#define ACC_SM_COUNT 148

template <class T> struct acc_bits { static const int value = (int)sizeof(T) * 8; };
template <class T> struct acc_unsigned;
template <> struct acc_unsigned<i8> { typedef u8 type; };
template <> struct acc_unsigned<i16> { typedef u16 type; };
template <> struct acc_unsigned<i32> { typedef u32 type; };
template <> struct acc_unsigned<i64> { typedef u64 type; };
template <> struct acc_unsigned<u8> { typedef u8 type; };
template <> struct acc_unsigned<u16> { typedef u16 type; };
template <> struct acc_unsigned<u32> { typedef u32 type; };
template <> struct acc_unsigned<u64> { typedef u64 type; };
template <class T> struct acc_is_signed { static const bool value = ((T)-1) < (T)0; };

// Status word of the context that launched the kernel.  Scalar helpers have no parameter block at
// hand, so the host stores the word's address here when it loads the module (the variable is absent
// from modules that never raise).  Codes: 1002 divide by zero, 1003 index out of bounds.
extern "C" { __device__ int* acc_status_word = nullptr; }
__device__ __forceinline__ void acc_raise(int code) {
  int* w = acc_status_word;
  if (w) atomicCAS(w, 0, code);
}

// quot/rem truncate toward zero; div/mod floor (Interpreter.hs:1328-1344).  Division by zero raises
// an exception in the reference (GHC's DivideByZero); here it is recorded in the status word (the
// call that next synchronises reports B200_ERR_ARITH) and the operation yields 0.
template <class T> __device__ __forceinline__ T acc_quot(T a, T b) {
  typedef typename acc_unsigned<T>::type U;
  if (b == 0) { acc_raise(1002); return 0; }
  if (acc_is_signed<T>::value && b == (T)-1) return (T)((U)0 - (U)a);
  return (T)(a / b);
}
template <class T> __device__ __forceinline__ T acc_rem(T a, T b) {
  if (b == 0) { acc_raise(1002); return 0; }
  if (acc_is_signed<T>::value && b == (T)-1) return 0;
  return (T)(a % b);
}
template <class T> __device__ __forceinline__ T acc_div(T a, T b) {
  T q = acc_quot<T>(a, b);
  if (acc_is_signed<T>::value) {
    T r = acc_rem<T>(a, b);
    if (r != 0 && ((r < 0) != (b < 0))) q = (T)(q - 1);
  }
  return q;
}
template <class T> __device__ __forceinline__ T acc_mod(T a, T b) {
  T r = acc_rem<T>(a, b);
  if (acc_is_signed<T>::value) {
    if (r != 0 && ((r < 0) != (b < 0))) r = (T)(r + b);
  }
  return r;
}
// shifts by >= the bit width are defined: 0, or the sign for arithmetic right shifts
template <class T> __device__ __forceinline__ T acc_shl(T a, i64 n) {
  typedef typename acc_unsigned<T>::type U;
  if (n < 0 || n >= acc_bits<T>::value) return 0;
  return (T)((U)((U)a << (int)n));
}
template <class T> __device__ __forceinline__ T acc_shr(T a, i64 n) {
  if (n < 0) return 0;
  if (n >= acc_bits<T>::value) return acc_is_signed<T>::value ? (T)(a < 0 ? -1 : 0) : (T)0;
  return (T)(a >> (int)n);
}
template <class T> __device__ __forceinline__ T acc_rotl(T a, i64 n) {
  typedef typename acc_unsigned<T>::type U;
  const int b = acc_bits<T>::value;
  int r = (int)(n % b);
  if (r < 0) r += b;
  if (r == 0) return a;
  U v = (U)a;
  return (T)(U)((U)(v << r) | (U)(v >> (b - r)));
}
template <class T> __device__ __forceinline__ i64 acc_popcount(T a) {
  typedef typename acc_unsigned<T>::type U;
  return (i64)__popcll((u64)(U)a);
}
template <class T> __device__ __forceinline__ i64 acc_clz(T a) {
  typedef typename acc_unsigned<T>::type U;
  return (i64)__clzll((long long)(u64)(U)a) - (64 - acc_bits<T>::value);
}
template <class T> __device__ __forceinline__ i64 acc_ctz(T a) {
  typedef typename acc_unsigned<T>::type U;
  const u64 v = (u64)(U)a;
  return v == 0 ? (i64)acc_bits<T>::value : (i64)(__ffsll((long long)v) - 1);
}
template <class F> __device__ __forceinline__ i64 acc_f2i(F x) { return (i64)x; }

// ---- warp shuffles of one scalar -------------------------------------------------
#define ACC_SHFL1(NAME, INTR)                                                                               \
  __device__ __forceinline__ i32 acc_shfl1_##NAME(i32 v, int d) { return INTR(ACC_FULL_MASK, v, d); }       \
  __device__ __forceinline__ u32 acc_shfl1_##NAME(u32 v, int d) { return INTR(ACC_FULL_MASK, v, d); }       \
  __device__ __forceinline__ i64 acc_shfl1_##NAME(i64 v, int d) { return INTR(ACC_FULL_MASK, v, d); }       \
  __device__ __forceinline__ u64 acc_shfl1_##NAME(u64 v, int d) { return INTR(ACC_FULL_MASK, v, d); }       \
  __device__ __forceinline__ f32 acc_shfl1_##NAME(f32 v, int d) { return INTR(ACC_FULL_MASK, v, d); }       \
  __device__ __forceinline__ f64 acc_shfl1_##NAME(f64 v, int d) { return INTR(ACC_FULL_MASK, v, d); }       \
  __device__ __forceinline__ i8 acc_shfl1_##NAME(i8 v, int d) { return (i8)INTR(ACC_FULL_MASK, (i32)v, d); } \
  __device__ __forceinline__ u8 acc_shfl1_##NAME(u8 v, int d) { return (u8)INTR(ACC_FULL_MASK, (u32)v, d); } \
  __device__ __forceinline__ i16 acc_shfl1_##NAME(i16 v, int d) { return (i16)INTR(ACC_FULL_MASK, (i32)v, d); } \
  __device__ __forceinline__ u16 acc_shfl1_##NAME(u16 v, int d) { return (u16)INTR(ACC_FULL_MASK, (u32)v, d); }
ACC_SHFL1(down, __shfl_down_sync)
ACC_SHFL1(up, __shfl_up_sync)
ACC_SHFL1(idx, __shfl_sync)

// ---- four consecutive elements: one 128-bit access per 16 bytes --------------------
// The address must be aligned to 4 * sizeof(T).  Loads go through the read-only
// path (inputs are never written by the kernel that reads them).
// Vector loads of stream operands: read-only path by default; kernels that read every element once and
// gain from it (the folds: +5 % for segmented folds) ask for the streaming, evict-first form.  The rank-2
// stencil must not: its neighbouring warps and its next application re-read what a warp loaded (-20 %).
#if defined(ACC_STREAM_LOADS) && ACC_STREAM_LOADS
#define ACC_LDV(ptr) __ldcs(ptr)
#else
#define ACC_LDV(ptr) __ldg(ptr)
#endif
template <class T, int BYTES> struct acc_vec4;
template <class T> struct acc_vec4<T, 4> {
  static __device__ __forceinline__ void ld(const T* p, T (&o)[4]) {
    const uint4 v = ACC_LDV(reinterpret_cast<const uint4*>(p));
    const u32 w[4] = {v.x, v.y, v.z, v.w};
    _Pragma("unroll") for (int k = 0; k < 4; ++k) o[k] = *reinterpret_cast<const T*>(&w[k]);
  }
  static __device__ __forceinline__ void st(T* p, const T (&o)[4]) {
    uint4 v;
    v.x = *reinterpret_cast<const u32*>(&o[0]);
    v.y = *reinterpret_cast<const u32*>(&o[1]);
    v.z = *reinterpret_cast<const u32*>(&o[2]);
    v.w = *reinterpret_cast<const u32*>(&o[3]);
    *reinterpret_cast<uint4*>(p) = v;
  }
};
template <class T> struct acc_vec4<T, 8> {
  static __device__ __forceinline__ void ld(const T* p, T (&o)[4]) {
    const ulonglong2 a = ACC_LDV(reinterpret_cast<const ulonglong2*>(p));
    const ulonglong2 b = ACC_LDV(reinterpret_cast<const ulonglong2*>(p) + 1);
    const u64 w[4] = {a.x, a.y, b.x, b.y};
    _Pragma("unroll") for (int k = 0; k < 4; ++k) o[k] = *reinterpret_cast<const T*>(&w[k]);
  }
  static __device__ __forceinline__ void st(T* p, const T (&o)[4]) {
    ulonglong2 a, b;
    a.x = *reinterpret_cast<const u64*>(&o[0]);
    a.y = *reinterpret_cast<const u64*>(&o[1]);
    b.x = *reinterpret_cast<const u64*>(&o[2]);
    b.y = *reinterpret_cast<const u64*>(&o[3]);
    reinterpret_cast<ulonglong2*>(p)[0] = a;
    reinterpret_cast<ulonglong2*>(p)[1] = b;
  }
};
template <class T> struct acc_vec4<T, 2> {
  static __device__ __forceinline__ void ld(const T* p, T (&o)[4]) {
    const uint2 v = ACC_LDV(reinterpret_cast<const uint2*>(p));
    const u16 w[4] = {(u16)(v.x & 0xffffu), (u16)(v.x >> 16), (u16)(v.y & 0xffffu), (u16)(v.y >> 16)};
    _Pragma("unroll") for (int k = 0; k < 4; ++k) o[k] = (T)w[k];
  }
  static __device__ __forceinline__ void st(T* p, const T (&o)[4]) {
    uint2 v;
    v.x = (u32)(u16)o[0] | ((u32)(u16)o[1] << 16);
    v.y = (u32)(u16)o[2] | ((u32)(u16)o[3] << 16);
    *reinterpret_cast<uint2*>(p) = v;
  }
};
template <class T> struct acc_vec4<T, 1> {
  static __device__ __forceinline__ void ld(const T* p, T (&o)[4]) {
    const u32 v = ACC_LDV(reinterpret_cast<const u32*>(p));
    _Pragma("unroll") for (int k = 0; k < 4; ++k) o[k] = (T)(u8)(v >> (8 * k));
  }
  static __device__ __forceinline__ void st(T* p, const T (&o)[4]) {
    *reinterpret_cast<u32*>(p) = (u32)(u8)o[0] | ((u32)(u8)o[1] << 8) | ((u32)(u8)o[2] << 16) | ((u32)(u8)o[3] << 24);
  }
};
template <class T> __device__ __forceinline__ void acc_ld4(const T* p, T (&o)[4]) { acc_vec4<T, (int)sizeof(T)>::ld(p, o); }
template <class T> __device__ __forceinline__ void acc_st4(T* p, const T (&o)[4]) { acc_vec4<T, (int)sizeof(T)>::st(p, o); }

// four consecutive elements from shared memory (address aligned to 4 * sizeof(T))
template <class T, int BYTES> struct acc_lds4_impl {
  static __device__ __forceinline__ void ld(const T* p, T (&o)[4]) {
    struct __align__(sizeof(T) * 4) quad { T v[4]; };
    const quad q = *reinterpret_cast<const quad*>(p);
    _Pragma("unroll") for (int k = 0; k < 4; ++k) o[k] = q.v[k];
  }
};
// 8-byte elements: neighbouring lanes are 32 bytes apart, so two plain 16-byte reads per lane would hit every
// bank twice.  The two halves are read in an order that alternates every four lanes: the eight lanes that are
// served together then cover all 32 banks once.  (Callers pass addresses that grow or shrink by 32 bytes per lane.)
template <class T> struct acc_lds4_impl<T, 8> {
  static __device__ __forceinline__ void ld(const T* p, T (&o)[4]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
    const int h = (threadIdx.x >> 2) & 1;
    const uint4 a = q[h], b = q[h ^ 1];
    const uint4 lo = h ? b : a, hi = h ? a : b;
    memcpy(&o[0], &lo, 16);
    memcpy(&o[2], &hi, 16);
  }
};
template <class T> __device__ __forceinline__ void acc_lds4(const T* p, T (&o)[4]) { acc_lds4_impl<T, (int)sizeof(T)>::ld(p, o); }

// Record the first device-side failure (a bounded wait that gave up, ...).
__device__ __forceinline__ void acc_fail(i64 err_ptr, int code) {
  atomicCAS(reinterpret_cast<int*>(err_ptr), 0, code);
}
