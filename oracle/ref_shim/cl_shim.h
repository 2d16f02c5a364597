/*
 * Shim that lets the reference's OpenCL C kernel sources compile as plain C99 --
 * TEST INFRASTRUCTURE ONLY (see oracle/ref_shim/ref_driver.c).
 *
 * The kernel files themselves are never copied: ref_driver.c #includes them in
 * place from the read-only reference checkout at build time.
 */
#ifndef DR_CL_SHIM_H
#define DR_CL_SHIM_H
#include <float.h>
#include <math.h>
#include <stddef.h>

#define __kernel
#define __global
#define __local
#define __constant const
#define __private
#define CLK_LOCAL_MEM_FENCE 1
#define CLK_GLOBAL_MEM_FENCE 2

size_t get_global_id(unsigned d);
size_t get_local_id(unsigned d);
size_t get_group_id(unsigned d);
size_t get_local_size(unsigned d);
size_t get_global_size(unsigned d);
size_t get_num_groups(unsigned d);
void barrier(int flags);

#define clamp(v, lo, hi) ((v) < (lo) ? (lo) : ((v) > (hi) ? (hi) : (v)))
#define mad(a, b, c) ((a) * (b) + (c))
#define mad24(a, b, c) ((a) * (b) + (c))
#define mul24(a, b) ((a) * (b))
#ifndef max
#define max(a, b) ((a) > (b) ? (a) : (b))
#endif
#ifndef min
#define min(a, b) ((a) < (b) ? (a) : (b))
#endif
#endif
