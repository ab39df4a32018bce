/*
 * Host-side stand-ins for the CUDA built-ins the reference kernels use, so that the
 * reference project's own .cu sources can be compiled by g++ and executed one logical
 * thread at a time on CPU cores.  Test infrastructure only.
 *
 * The reference kernels never synchronise or communicate between threads (no
 * __syncthreads, shuffles or atomics), and every __shared__ array is indexed by
 * threadIdx.x first, so running the threads of a block one after another on one CPU
 * thread preserves their semantics.
 */
#pragma once
#include <math.h>
#include <stddef.h>

struct cfshim_dim3 { unsigned int x, y, z; };
static thread_local cfshim_dim3 threadIdx, blockIdx, blockDim, gridDim;

#define __global__
#define __device__
#define __host__
#define __forceinline__ inline
#define __shared__ static thread_local
#define __restrict__

static inline int max(int a, int b) { return a > b ? a : b; }
static inline int min(int a, int b) { return a < b ? a : b; }
static inline float max(float a, float b) { return fmaxf(a, b); }
static inline float min(float a, float b) { return fminf(a, b); }
/* CUDA's mixed overloads promote to double */
static inline double max(float a, double b) { return fmax((double)a, b); }
static inline double max(double a, float b) { return fmax(a, (double)b); }
static inline double min(float a, double b) { return fmin((double)a, b); }
static inline double min(double a, float b) { return fmin(a, (double)b); }
static inline double max(double a, double b) { return fmax(a, b); }
static inline double min(double a, double b) { return fmin(a, b); }
static inline long long max(long long a, long long b) { return a > b ? a : b; }
static inline long long min(long long a, long long b) { return a < b ? a : b; }

static inline void cfshim_set(unsigned int b, unsigned int t, unsigned int grid, unsigned int block)
{
    blockIdx.x = b; blockIdx.y = blockIdx.z = 0;
    threadIdx.x = t; threadIdx.y = threadIdx.z = 0;
    blockDim.x = block; blockDim.y = blockDim.z = 1;
    gridDim.x = grid; gridDim.y = gridDim.z = 1;
}
