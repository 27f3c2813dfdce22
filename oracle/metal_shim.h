// TEST INFRASTRUCTURE — not part of the product.
//
// Minimal shim that lets the reference's Metal Shading Language kernels for
// distances, k-means and scalar quantisation compile as host C++, so that the
// reference's own shader arithmetic can be executed on the CPU and used to pin
// the restatement in cpu_ref.cpp.  The shader text itself is read from the
// reference tree at build time (see Makefile) and is never stored here.
//
// MSL has no double type: an unsuffixed literal such as 1e-8 is a float, so the
// translation unit must be built with -fsingle-precision-constant, and with
// -ffp-contract=off so that sums are rounded after every operation.
#pragma once
#include <algorithm>
#include <cmath>
#include <cstdint>

namespace metal {}
#define kernel
#define constant const
#define device
#define threadgroup
#define memory_order_relaxed 0
typedef unsigned int uint;
typedef unsigned char uchar;
struct uint2 { uint x, y; };
typedef float atomic_float;
typedef uint atomic_uint;
template <class T, class U> static inline T atomic_fetch_add_explicit(T* p, U v, int) { T o = *p; *p = o + (T)v; return o; }
template <class T, class U> static inline void atomic_store_explicit(T* p, U v, int) { *p = (T)v; }
using std::sqrt;
using std::abs;
using std::round;
static inline float min(float a, float b) { return b < a ? b : a; }
static inline float max(float a, float b) { return a < b ? b : a; }
static inline uint min(uint a, uint b) { return b < a ? b : a; }
static inline float clamp(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }
