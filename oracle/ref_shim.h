/* Host execution model for the reference's OpenCL-C GEMM kernels. TEST INFRASTRUCTURE ONLY.
 *
 * oracle/build_ref.py pastes the bodies of the reference's kernel files (read where they lie in the reference
 * tree, never copied into this repository) after this header and compiles the result as C (OpenCL C is a C99
 * dialect) once per precision. The header supplies what an OpenCL device would: work-item and work-group ids,
 * barrier(), address-space keywords, vector types, and one launcher that runs a grid work-group by work-group.
 * Work-items of a group are fibers (ucontext) resumed round-robin; barrier() yields, so every work-item of the
 * group reaches a barrier before any passes it. `__local` becomes `static`: one group runs at a time on one
 * thread, so a function-local static array is exactly the group's local memory. */
#pragma once

#include <math.h>
#include <stdbool.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <ucontext.h>

typedef struct {
  int local_id[3];
  int group_id[3];
  int local_size[3];
  int num_groups[3];
} refshim_work_item;

static refshim_work_item* volatile refshim_current = NULL;
static ucontext_t refshim_scheduler;
static ucontext_t* volatile refshim_fiber = NULL;
static void (*refshim_body)(void*) = NULL;
static void* refshim_body_arg = NULL;
static volatile int* volatile refshim_done_flag = NULL;

static void refshim_fiber_entry(void) {
  refshim_body(refshim_body_arg);
  *refshim_done_flag = 1;
  swapcontext(refshim_fiber, &refshim_scheduler);
}

/* Runs body(arg) once per work-item of a (gx, gy, gz) x (lx, ly, lz) launch. Returns 0, or -1 on allocation failure. */
static int refshim_run_grid(const int groups[3], const int local[3], void (*body)(void*), void* arg) {
  const int per_group = local[0] * local[1] * local[2];
  const size_t stack_bytes = 256 * 1024;
  ucontext_t* ctx = (ucontext_t*)malloc(sizeof(ucontext_t) * per_group);
  refshim_work_item* items = (refshim_work_item*)malloc(sizeof(refshim_work_item) * per_group);
  char* stacks = (char*)malloc(stack_bytes * per_group);
  char* done = (char*)malloc(per_group);
  if (!ctx || !items || !stacks || !done) return -1;
  refshim_body = body;
  refshim_body_arg = arg;
  for (int gz = 0; gz < groups[2]; ++gz)
    for (int gy = 0; gy < groups[1]; ++gy)
      for (int gx = 0; gx < groups[0]; ++gx) {
        for (int i = 0; i < per_group; ++i) {
          refshim_work_item* w = &items[i];
          w->local_id[0] = i % local[0];
          w->local_id[1] = (i / local[0]) % local[1];
          w->local_id[2] = i / (local[0] * local[1]);
          w->group_id[0] = gx; w->group_id[1] = gy; w->group_id[2] = gz;
          for (int d = 0; d < 3; ++d) { w->local_size[d] = local[d]; w->num_groups[d] = groups[d]; }
          getcontext(&ctx[i]);
          ctx[i].uc_stack.ss_sp = stacks + stack_bytes * i;
          ctx[i].uc_stack.ss_size = stack_bytes;
          ctx[i].uc_link = &refshim_scheduler;
          makecontext(&ctx[i], refshim_fiber_entry, 0);
          done[i] = 0;
        }
        int remaining = per_group;
        while (remaining > 0) {
          for (int i = 0; i < per_group; ++i) {
            if (done[i]) continue;
            volatile int finished = 0;
            refshim_current = &items[i];
            refshim_fiber = &ctx[i];
            refshim_done_flag = &finished;
            swapcontext(&refshim_scheduler, &ctx[i]);
            if (finished) { done[i] = 1; --remaining; }
          }
        }
      }
  free(ctx); free(items); free(stacks); free(done);
  return 0;
}

static inline void refshim_barrier(void) { swapcontext(refshim_fiber, &refshim_scheduler); }

static inline int get_local_id(int d) { return refshim_current->local_id[d]; }
static inline int get_group_id(int d) { return refshim_current->group_id[d]; }
static inline int get_local_size(int d) { return refshim_current->local_size[d]; }
static inline int get_num_groups(int d) { return refshim_current->num_groups[d]; }
static inline int get_global_size(int d) { return get_num_groups(d) * get_local_size(d); }
static inline int get_global_id(int d) { return get_group_id(d) * get_local_size(d) + get_local_id(d); }

#define CLK_LOCAL_MEM_FENCE 1
#define CLK_GLOBAL_MEM_FENCE 2
#define barrier(flags) refshim_barrier()

#define __kernel
#define __global
#define __constant const
#define __local static
#define LOCAL_PTR
#define RELAX_WORKGROUP_SIZE 1

typedef _Float16 half;
#define REFSHIM_VECTORS(T)                                                                   \
  typedef struct { T x, y; } T##2;                                                           \
  typedef struct { T x, y, z, w; } T##4;                                                     \
  typedef struct { T s0, s1, s2, s3, s4, s5, s6, s7; } T##8;                                 \
  typedef struct { T s0, s1, s2, s3, s4, s5, s6, s7, s8, s9, sA, sB, sC, sD, sE, sF; } T##16;
REFSHIM_VECTORS(half)
REFSHIM_VECTORS(float)
REFSHIM_VECTORS(double)

/* OpenCL built-ins the im2col / col2im kernels use on ints. */
static inline int refshim_min(int a, int b) { return a < b ? a : b; }
static inline int refshim_max(int a, int b) { return a > b ? a : b; }
#define min(a, b) refshim_min((a), (b))
#define max(a, b) refshim_max((a), (b))
