/*
 * Stand-in for <curand_kernel.h> in the CPU build of the reference kernels.  The CPU
 * build fixes SYMM_BREAK_NOISE to 0, so the drawn value is multiplied by zero and
 * only has to be finite.
 */
#pragma once
struct curandState { unsigned int pad[12]; };
static inline void curand_init(unsigned long long, unsigned long long, unsigned long long, curandState*) {}
static inline float curand_uniform(curandState*) { return 0.5f; }
