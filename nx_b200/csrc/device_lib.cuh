// Device-side support library for the fused kernels the planner generates.
//
// This text is compiled together with each generated kernel body (NVRTC,
// sm_100a), so it uses no headers: fixed-width types, bf16/f16 conversions,
// the math routines, 128-bit vector access and the row reductions are all
// defined here.  Numerics contract:
//   * f32 functions are accurate to a few ulp (parity tolerance is rtol 1e-5);
//   * bf16/f16 values are held widened in a float register and rounded to
//     nearest-even after every graph node (what a literal reading of the
//     user's graph asks for);
//   * integer arithmetic wraps.
#pragma once

typedef signed char int8_t;
typedef unsigned char uint8_t;
typedef short int16_t;
typedef unsigned short uint16_t;
typedef int int32_t;
typedef unsigned int uint32_t;
typedef long long int64_t;
typedef unsigned long long uint64_t;

#define NXB_DEV __device__ __forceinline__
#define NXB_INF __int_as_float(0x7f800000)
#define NXB_NAN __int_as_float(0x7fc00000)

// ---- storage types for the 16-bit floats -----------------------------------------
struct bf16_t { uint16_t bits; };
struct f16_t { uint16_t bits; };

NXB_DEV float bf16_to_f32(bf16_t h) { return __uint_as_float(((uint32_t)h.bits) << 16); }
NXB_DEV bf16_t f32_to_bf16(float f) {
  bf16_t r;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r.bits) : "f"(f));
  return r;
}
// round a float register to the nearest bf16 value, keeping it widened
NXB_DEV float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }
NXB_DEV float f16_to_f32(f16_t h) {
  float f;
  asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h.bits));
  return f;
}
NXB_DEV f16_t f32_to_f16(float f) {
  f16_t r;
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(r.bits) : "f"(f));
  return r;
}
NXB_DEV float round_f16(float f) { return f16_to_f32(f32_to_f16(f)); }

// ---- memory <-> register representation -----------------------------------------
// Storage type S (what sits in HBM) and register type R (what code computes on).
template <typename S> struct Repr { typedef S R; static NXB_DEV R load(S s) { return s; } static NXB_DEV S store(R r) { return r; } };
template <> struct Repr<bf16_t> { typedef float R; static NXB_DEV float load(bf16_t s) { return bf16_to_f32(s); } static NXB_DEV bf16_t store(float r) { return f32_to_bf16(r); } };
template <> struct Repr<f16_t> { typedef float R; static NXB_DEV float load(f16_t s) { return f16_to_f32(s); } static NXB_DEV f16_t store(float r) { return f32_to_f16(r); } };

template <typename S, int V> struct __align__(sizeof(S) * V) Pack { S v[V]; };

// Vector load of V consecutive elements (address must be aligned to sizeof(S)*V).
template <typename S, int V>
NXB_DEV void ld_vec(const S* __restrict__ p, typename Repr<S>::R (&dst)[V]) {
  Pack<S, V> t = *reinterpret_cast<const Pack<S, V>*>(p);
#pragma unroll
  for (int i = 0; i < V; ++i) dst[i] = Repr<S>::load(t.v[i]);
}
template <typename S, int V>
NXB_DEV void st_vec(S* __restrict__ p, const typename Repr<S>::R (&src)[V]) {
  Pack<S, V> t;
#pragma unroll
  for (int i = 0; i < V; ++i) t.v[i] = Repr<S>::store(src[i]);
#if defined(NXB_STREAMING_STORES)
  // results larger than the cache, read by nobody soon: evict-first (the planner defines this per kernel)
  if constexpr (sizeof(Pack<S, V>) == 16) {
    const uint4 w = *reinterpret_cast<const uint4*>(&t);
    asm volatile("st.global.cs.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w) : "memory");
    return;
  }
#endif
  *reinterpret_cast<Pack<S, V>*>(p) = t;
}
template <typename S> NXB_DEV typename Repr<S>::R ld1(const S* __restrict__ p) { return Repr<S>::load(*p); }
template <typename S> NXB_DEV void st1(S* __restrict__ p, typename Repr<S>::R v) { *p = Repr<S>::store(v); }

// ---- conversions (as_type) ---------------------------------------------------------
// float -> integer: truncate; NaN -> 0; out of range (incl. +-inf) saturates.
template <typename I> NXB_DEV I f2i(double f) {
  const bool is_signed = ((I)-1) < (I)0;
  const int bits = sizeof(I) * 8;
  if (f != f) return (I)0;
  if (is_signed) {
    double lo = -__longlong_as_double(0x3ff0000000000000LL + ((long long)(bits - 1) << 52));  // -2^(bits-1)
    if (f <= lo) return (I)((uint64_t)1 << (bits - 1));
    if (f >= -lo) return (I)(((uint64_t)1 << (bits - 1)) - 1);
    return (I)(long long)f;
  } else {
    if (f <= 0.0) return (I)0;
    double hi = __longlong_as_double(0x3ff0000000000000LL + ((long long)bits << 52));          // 2^bits
    if (f >= hi) return (I)~(I)0;
    return (I)(unsigned long long)f;
  }
}

// ---- f32 math ------------------------------------------------------------------------
NXB_DEV float fast_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
NXB_DEV float fast_rcp(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
NXB_DEV float fast_lg2(float x) { float y; asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

// exp(x) in ~6 instructions at ~2 ulp.  MUFU.EX2 is accurate to 2^-22 for any
// argument, so the only error to remove is the one made when x*log2(e) is
// rounded to f32 (its ulp grows with |x|): the rounding error of the product
// and the representation error of the constant are recovered with two FMAs and
// applied as a first-order correction, exp2(t + c) = exp2(t) * (1 + c ln 2).
NXB_DEV float nx_exp(float x) {
  const float L2E = 1.44269502162933349609375f;        // f32(log2 e)
  const float L2E_LO = 1.925963033500665e-08f;          // log2 e - f32(log2 e)
  float t = x * L2E;
  float c = fmaf(x, L2E, -t);
  c = fmaf(x, L2E_LO, c);
  float p = fast_ex2(t);
  float r = fmaf(p * c, 0.693147182464599609375f, p);
  // p is 0 or inf at the ends of the range (and for infinite x, where c is NaN): return it as is
  return (p == 0.f || p == NXB_INF) ? p : r;
}
// 1 / (1 + exp(-x)); rcp.approx is within 1 ulp.  The exponential here needs no compensated
// product: its relative error (|x| log2(e) 2^-24 + 2 ulp of ex2, < 8e-6 over the finite range) only
// matters where it dominates the sum, and ex2's own 0 / inf ends give the right limits.
NXB_DEV float nx_sigmoid(float x) { return fast_rcp(1.f + fast_ex2(x * -1.44269502162933349609375f)); }
// tanh: odd polynomial near 0 (keeps relative accuracy), 1 - 2/(exp(2|x|)+1) elsewhere
NXB_DEV float nx_tanh(float x) {
  const float ax = fabsf(x);
  const float x2 = x * x;
  float p = 0.021869488f;                 // 62/2835
  p = fmaf(p, x2, -0.053968254f);         // -17/315
  p = fmaf(p, x2, 0.133333333f);          // 2/15
  p = fmaf(p, x2, -0.333333333f);         // -1/3
  const float small = fmaf(p * x2, x, x);
  const float e = fast_ex2(ax * 2.8853900432586669921875f);     // exp(2|x|): an error of 1e-5 in e moves the result by < 5e-6 of it
  float big = fmaf(-2.f, fast_rcp(e + 1.f), 1.f);
  big = copysignf(big, x);
  return (ax < 0.12f) ? small : big;
}
NXB_DEV float nx_log(float x) { return logf(x); }
NXB_DEV float nx_rsqrt(float x) { return 1.0f / sqrtf(x); }
NXB_DEV float nx_erf_inv(float x) { return erfinvf(x); }
NXB_DEV float nx_round(float x) { return roundf(x); }     // half away from zero
NXB_DEV double nx_round(double x) { return round(x); }
NXB_DEV float nx_sign(float x) { return (x > 0.f) ? 1.f : ((x < 0.f) ? -1.f : x); }
NXB_DEV double nx_sign(double x) { return (x > 0.0) ? 1.0 : ((x < 0.0) ? -1.0 : x); }
template <typename I> NXB_DEV I nx_sign_i(I x) { return (I)((x > 0) - (x < 0)); }

NXB_DEV double nx_exp(double x) { return exp(x); }
NXB_DEV double nx_sigmoid(double x) { return 1.0 / (1.0 + exp(-x)); }
NXB_DEV double nx_tanh(double x) { return tanh(x); }
NXB_DEV double nx_log(double x) { return log(x); }
NXB_DEV double nx_rsqrt(double x) { return 1.0 / sqrt(x); }
NXB_DEV double nx_erf_inv(double x) { return erfinv(x); }

// max/min where NaN wins (nx element_max/element_min)
NXB_DEV float nx_max(float a, float b) { float r; asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }
NXB_DEV float nx_min(float a, float b) { float r; asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b)); return r; }
NXB_DEV double nx_max(double a, double b) { return (a != a || b != b) ? (double)NXB_NAN : fmax(a, b); }
NXB_DEV double nx_min(double a, double b) { return (a != a || b != b) ? (double)NXB_NAN : fmin(a, b); }
#define NXB_INT_MINMAX(T) \
  NXB_DEV T nx_max(T a, T b) { return a > b ? a : b; } \
  NXB_DEV T nx_min(T a, T b) { return a < b ? a : b; }
NXB_INT_MINMAX(int8_t) NXB_INT_MINMAX(uint8_t) NXB_INT_MINMAX(int16_t) NXB_INT_MINMAX(uint16_t)
NXB_INT_MINMAX(int32_t) NXB_INT_MINMAX(uint32_t) NXB_INT_MINMAX(int64_t) NXB_INT_MINMAX(uint64_t)

template <typename I> NXB_DEV I nx_ipow(I base, I e) {
  I r = 1;
  const bool is_signed = ((I)-1) < (I)0;
  if (is_signed && e < 0) return (base == 1) ? (I)1 : ((base == (I)-1) ? ((e & 1) ? (I)-1 : (I)1) : (I)0);
  while (e) { if (e & 1) r = (I)(r * base); base = (I)(base * base); e = (I)((uint64_t)e >> 1); }
  return r;
}
template <typename I> NXB_DEV I nx_idiv(I a, I b) { return b == 0 ? (I)-1 : (I)(a / b); }
template <typename I> NXB_DEV I nx_irem(I a, I b) { return b == 0 ? a : (I)(a % b); }
template <typename I> NXB_DEV I nx_shl(I a, I b) { return ((uint64_t)b >= sizeof(I) * 8) ? (I)0 : (I)(a << b); }
template <typename I> NXB_DEV I nx_shr(I a, I b) {
  const bool is_signed = ((I)-1) < (I)0;
  if ((uint64_t)b >= sizeof(I) * 8) return (is_signed && a < 0) ? (I)-1 : (I)0;
  return (I)(a >> b);
}
template <typename I> NXB_DEV I nx_popc(I a) {
  return (I)__popcll((unsigned long long)a & (sizeof(I) == 8 ? ~0ULL : ((1ULL << (sizeof(I) * 8 % 64)) - 1)));
}
template <typename I> NXB_DEV I nx_clz(I a) {
  unsigned long long u = (unsigned long long)a & (sizeof(I) == 8 ? ~0ULL : ((1ULL << (sizeof(I) * 8 % 64)) - 1));
  return (I)(__clzll((long long)u) - (64 - (int)sizeof(I) * 8));
}

// ---- row staging: bulk copy of the next row into shared memory while this one is computed ----
NXB_DEV uint32_t stg_smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
NXB_DEV void stg_bar_init(void* bar) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(stg_smem_addr(bar)) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
NXB_DEV void stg_expect(void* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(stg_smem_addr(bar)), "r"(bytes) : "memory");
}
// 1-D bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion on `bar`
NXB_DEV void stg_copy(void* dst, const void* src, uint32_t bytes, void* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(stg_smem_addr(dst)), "l"(src), "r"(bytes), "r"(stg_smem_addr(bar)) : "memory");
}
NXB_DEV bool stg_try_wait(void* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(stg_smem_addr(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait (about one second).  On expiry the caller stops using the staging buffer and
// reads the row from global memory instead, so a lost copy costs speed, never correctness.
NXB_DEV bool stg_wait(void* bar, uint32_t parity) {
  if (stg_try_wait(bar, parity)) return true;
  // the SM cycle counter is cheap to read; the global nanosecond timer is not
  const long long t0 = clock64();
  for (;;) {
    for (int i = 0; i < 32; ++i) if (stg_try_wait(bar, parity)) return true;
    if (clock64() - t0 > 2000000000ll) return false;
  }
}

// An index or a slice start clamped into [0, n - 1] (gather, dynamic slice, put_slice); works for
// every integer type an index tensor may have, unsigned 64-bit included.
template <typename T> NXB_DEV long long nx_clamp_index(T v, long long n) {
  if (v < (T)0) return 0;
  if ((unsigned long long)v > (unsigned long long)(n - 1)) return n - 1;
  return (long long)v;
}

// ---- reductions ------------------------------------------------------------------------
// Combine operators.  Each has ::apply(a, b) on the register type.
struct OpSum { template <typename T> static NXB_DEV T apply(T a, T b) { return a + b; } };
struct OpProd { template <typename T> static NXB_DEV T apply(T a, T b) { return a * b; } };
struct OpMax { template <typename T> static NXB_DEV T apply(T a, T b) { return nx_max(a, b); } };
struct OpMin { template <typename T> static NXB_DEV T apply(T a, T b) { return nx_min(a, b); } };
struct OpAnd { template <typename T> static NXB_DEV T apply(T a, T b) { return (T)(a & b); } };
struct OpOr { template <typename T> static NXB_DEV T apply(T a, T b) { return (T)(a | b); } };

template <typename T> NXB_DEV T shfl_xor(T v, int m) {
  if (sizeof(T) == 8) {
    long long x = *reinterpret_cast<long long*>(&v);
    x = __shfl_xor_sync(0xffffffffu, x, m);
    return *reinterpret_cast<T*>(&x);
  } else if (sizeof(T) == 4) {
    int x = *reinterpret_cast<int*>(&v);
    x = __shfl_xor_sync(0xffffffffu, x, m);
    return *reinterpret_cast<T*>(&x);
  } else {
    int x = (int)v;
    x = __shfl_xor_sync(0xffffffffu, x, m);
    return (T)x;
  }
}

template <typename Op, typename T> NXB_DEV T warp_reduce(T v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v = Op::apply(v, shfl_xor(v, m));
  return v;
}

// All THREADS threads of the CTA cooperate on one row; every thread gets the result.
// `scratch` is shared memory with room for 32 elements of 8 bytes.
template <typename Op, typename T, int THREADS>
NXB_DEV T row_reduce(T v, void* scratch) {
  v = warp_reduce<Op>(v);
  if (THREADS > 32) {
    T* s = reinterpret_cast<T*>(scratch);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                    // scratch may still be read from the previous use
    if (lane == 0) s[warp] = v;
    __syncthreads();
    // every warp reduces the per-warp partials itself: one barrier fewer than a broadcast
    const int NW = THREADS / 32;
    T w = s[lane & (NW - 1)];          // every aligned group of NW lanes folds all partials
    if (NW < 32) {
#pragma unroll
      for (int m = NW / 2; m > 0; m >>= 1) w = Op::apply(w, shfl_xor(w, m));
    } else {
      w = warp_reduce<Op>(w);
    }
    v = w;
  }
  return v;
}

// Several reductions of one phase share a single pair of barriers: every warp reduces its own
// values with shuffles, lane 0 of each warp parks them in shared memory (one 32-entry, 8-byte
// slot array per reduction), and after the barrier every warp folds the per-warp partials.
template <typename T> NXB_DEV void park_partial(void* scratch, int slot, T v) {
  reinterpret_cast<T*>(reinterpret_cast<long long*>(scratch) + slot * 32)[threadIdx.x >> 5] = v;
}
template <typename Op, typename T, int THREADS> NXB_DEV T fold_partials(const void* scratch, int slot) {
  const int NW = THREADS / 32, lane = threadIdx.x & 31;
  T w = reinterpret_cast<const T*>(reinterpret_cast<const long long*>(scratch) + slot * 32)[lane & (NW - 1)];
#pragma unroll
  for (int m = NW / 2; m > 0; m >>= 1) w = Op::apply(w, shfl_xor(w, m));
  return w;
}

// (value, index) pair for argmax/argmin.  `better(a, b)` is a strict total
// order, so the result does not depend on the reduction tree:
//   * a NaN beats every number; among NaNs the highest index wins (what
//     Nx.BinaryBackend's left-to-right scan returns);
//   * otherwise the larger (argmax) / smaller (argmin) value wins;
//   * equal values: lowest index (tie_break :low) or highest (:high).
template <typename T> struct ArgPair { T v; long long i; };

template <typename T> NXB_DEV bool is_nan_any(T) { return false; }
template <> NXB_DEV bool is_nan_any<float>(float x) { return x != x; }
template <> NXB_DEV bool is_nan_any<double>(double x) { return x != x; }

template <bool IS_MAX, bool TIE_HIGH, typename T>
NXB_DEV bool arg_better(const ArgPair<T>& a, const ArgPair<T>& b) {
  if (b.i < 0) return a.i >= 0;
  if (a.i < 0) return false;
  const bool an = is_nan_any(a.v), bn = is_nan_any(b.v);
  if (an || bn) return an && (!bn || a.i > b.i);
  if (a.v != b.v) return IS_MAX ? (a.v > b.v) : (a.v < b.v);
  return TIE_HIGH ? (a.i > b.i) : (a.i < b.i);
}

// One step of a thread's own scan.  A thread visits its elements in increasing
// index order, so "replace when strictly better (or equal, for tie_break :high),
// or when the candidate is NaN" reproduces the order above without comparing indices.
template <bool IS_MAX, bool TIE_HIGH, typename T>
NXB_DEV void arg_step(ArgPair<T>& acc, T v, long long i) {
  bool take;
  if (TIE_HIGH) take = IS_MAX ? (v >= acc.v) : (v <= acc.v);
  else take = IS_MAX ? (v > acc.v) : (v < acc.v);
  // (an ordered comparison with a NaN accumulator is false by itself: a NaN, once taken, is only replaced by a later NaN)
  take = take || is_nan_any(v) || acc.i < 0;
  acc.v = take ? v : acc.v;
  acc.i = take ? i : acc.i;
}

template <bool IS_MAX, bool TIE_HIGH, typename T>
NXB_DEV ArgPair<T> arg_combine(ArgPair<T> a, ArgPair<T> b) { return arg_better<IS_MAX, TIE_HIGH>(b, a) ? b : a; }

template <bool IS_MAX, bool TIE_HIGH, typename T, int THREADS>
NXB_DEV ArgPair<T> row_arg_reduce(ArgPair<T> p, void* scratch) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) {
    ArgPair<T> o;
    o.v = shfl_xor(p.v, m);
    o.i = shfl_xor(p.i, m);
    p = arg_combine<IS_MAX, TIE_HIGH>(p, o);
  }
  if (THREADS > 32) {
    // scratch: 32 values (8 bytes each) followed by 32 indices
    long long* sv = reinterpret_cast<long long*>(scratch);
    long long* si = sv + 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) { T* pv = reinterpret_cast<T*>(&sv[warp]); *pv = p.v; si[warp] = p.i; }
    __syncthreads();
    const int NW = THREADS / 32;
    ArgPair<T> w;
    if (lane < NW) { w.v = *reinterpret_cast<T*>(&sv[lane]); w.i = si[lane]; } else { w.v = p.v; w.i = -1; }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
      ArgPair<T> o;
      o.v = shfl_xor(w.v, m);
      o.i = shfl_xor(w.i, m);
      w = arg_combine<IS_MAX, TIE_HIGH>(w, o);
    }
    p = w;
  }
  return p;
}

template <bool IS_MAX, bool TIE_HIGH, typename T> NXB_DEV ArgPair<T> warp_arg_reduce(ArgPair<T> p) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) {
    ArgPair<T> o;
    o.v = shfl_xor(p.v, m);
    o.i = shfl_xor(p.i, m);
    p = arg_combine<IS_MAX, TIE_HIGH>(p, o);
  }
  return p;
}
// an arg-reduction uses two slots: values in `slot`, indices in `slot + 1`
template <typename T> NXB_DEV void park_arg_partial(void* scratch, int slot, const ArgPair<T>& p) {
  park_partial<T>(scratch, slot, p.v);
  park_partial<long long>(scratch, slot + 1, p.i);
}
template <bool IS_MAX, bool TIE_HIGH, typename T, int THREADS>
NXB_DEV ArgPair<T> fold_arg_partials(const void* scratch, int slot) {
  const int NW = THREADS / 32, lane = threadIdx.x & 31;
  const long long* base = reinterpret_cast<const long long*>(scratch);
  ArgPair<T> w;
  w.v = reinterpret_cast<const T*>(base + slot * 32)[lane & (NW - 1)];
  w.i = (base + (slot + 1) * 32)[lane & (NW - 1)];
#pragma unroll
  for (int m = NW / 2; m > 0; m >>= 1) {
    ArgPair<T> o;
    o.v = shfl_xor(w.v, m);
    o.i = shfl_xor(w.i, m);
    w = arg_combine<IS_MAX, TIE_HIGH>(w, o);
  }
  return w;
}
