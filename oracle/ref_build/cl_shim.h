// OpenCL C -> C++ shim: just enough of the OpenCL C language for clDNN's reference
// kernels (fused_conv_eltwise_gpu_ref.cl, pooling_gpu_int8_ref.cl, ...) to compile
// unmodified with g++ and run one work-item at a time on the host.  TEST INFRASTRUCTURE.
// Built-ins follow the OpenCL C specification: round() = half away from zero,
// convert_<t>_sat(float) = NaN -> 0, clamp, truncate; fmax/fmin ignore a NaN operand.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstddef>
#include <climits>
#include <algorithm>

typedef unsigned int uint;
typedef unsigned char uchar;
typedef unsigned short ushort;
typedef unsigned long ulong;

#define __kernel
#define __global
#define __local
#define __constant const
#define __private
#define KERNEL(name) void name
#define FUNC(name) name
#define FUNC_CALL(name) name
#define CHAR_MIN_CL (-128)

static thread_local size_t cl_gid[3];
static inline size_t get_global_id(int d) { return cl_gid[d]; }

static inline float convert_float(float v) { return v; }
static inline float convert_float(int v) { return (float)v; }
static inline float convert_float(uint v) { return (float)v; }
static inline float convert_float(char v) { return (float)v; }
static inline float convert_float(uchar v) { return (float)v; }
static inline int convert_int(float v) { return (int)v; }
static inline int convert_int(int v) { return v; }
static inline int convert_int(char v) { return v; }
static inline int convert_int(uchar v) { return v; }
static inline char convert_char(int v) { return (char)v; }
static inline char convert_char(float v) { return (char)(int)v; }
static inline uchar convert_uchar(int v) { return (uchar)v; }
static inline uchar convert_uchar(float v) { return (uchar)(int)v; }

template <class T> static inline T cl_sat_from_float(float v, int lo, int hi)
{
    if (v != v) return (T)0;
    if (v <= (float)lo) return (T)lo;
    if (v >= (float)hi) return (T)hi;
    return (T)(int)v;
}
static inline char convert_char_sat(float v) { return cl_sat_from_float<char>(v, -128, 127); }
static inline char convert_char_sat(int v) { return (char)std::min(127, std::max(-128, v)); }
static inline char convert_char_sat(char v) { return v; }
static inline char convert_char_sat(uchar v) { return (char)std::min<int>(127, v); }
static inline uchar convert_uchar_sat(float v) { return cl_sat_from_float<uchar>(v, 0, 255); }
static inline uchar convert_uchar_sat(int v) { return (uchar)std::min(255, std::max(0, v)); }
static inline uchar convert_uchar_sat(uchar v) { return v; }
static inline uchar convert_uchar_sat(char v) { return (uchar)std::max<int>(0, v); }
static inline int convert_int_sat(int v) { return v; }
static inline int convert_int_sat(char v) { return v; }
static inline int convert_int_sat(uchar v) { return v; }
static inline int convert_int_sat(float v)
{
    if (v != v) return 0;
    if (v >= 2147483648.0f) return INT_MAX;
    if (v <= -2147483648.0f) return INT_MIN;
    return (int)v;
}

static inline float round(float v) { return ::roundf(v); }
static inline float fmax(float a, float b) { return ::fmaxf(a, b); }
static inline float fmin(float a, float b) { return ::fminf(a, b); }
static inline int max(int a, int b) { return a > b ? a : b; }
static inline int min(int a, int b) { return a < b ? a : b; }
static inline uint max(uint a, uint b) { return a > b ? a : b; }
static inline uint min(uint a, uint b) { return a < b ? a : b; }
static inline float native_exp(float v) { return ::expf(v); }
static inline bool isinf(float v) { return std::isinf(v); }
static inline bool isinf(int) { return false; }
