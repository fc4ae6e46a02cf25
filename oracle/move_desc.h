/* TEST INFRASTRUCTURE ONLY: one data-movement layer (Concat, Splitter, Permute, Transpose, StridedSlice, Slice) as the
 * reference's queue descriptors state it, for the CPU restatement (q8_oracle.c) and the binding over the real CpuRef
 * workloads (cpuref_capi.cpp).  Host pointers. */
#ifndef ORACLE_MOVE_DESC_H
#define ORACLE_MOVE_DESC_H
#include "../include/b200k.h"

enum { MOVE_CONCAT = 0, MOVE_SPLIT = 1, MOVE_PERMUTE = 2, MOVE_TRANSPOSE = 3, MOVE_STRIDED_SLICE = 4, MOVE_SLICE = 5,
       MOVE_DEPTH_TO_SPACE = 6, MOVE_SPACE_TO_DEPTH = 7,      /* perm[0] = block size, perm[1] = 1 for NCHW */
       MOVE_CHANNEL_SHUFFLE = 8,                              /* perm[0] = axis, perm[1] = groups */
       MOVE_STACK = 9,                                        /* perm[0] = axis; whole = the output, views = the inputs */
       MOVE_TILE = 12,                                        /* perm = multiples */
       MOVE_BROADCAST_TO = 13,                                /* view_shape[0] = the shape to broadcast to */
       MOVE_BATCH_TO_SPACE = 10, MOVE_SPACE_TO_BATCH = 11 };  /* perm[0] = 1 for NCHW; begin = block shape, end / stride =
                                                                 crops or padding before / after, per spatial dimension */

typedef struct {
    int32_t kind, rank;
    b200k_qtensor whole;            /* Concat: the output; every other kind: the input */
    int32_t whole_shape[6];
    int32_t n_views;                /* Concat: inputs; Splitter: outputs; others: 1 (the output) */
    b200k_qtensor view[8];
    int32_t view_rank[8];           /* 0: the rank of the whole tensor (a StridedSlice with shrunk axes has fewer) */
    int32_t view_shape[8][6];
    int32_t view_origin[8][6];      /* Concat / Splitter: ViewOrigin of each view */
    int32_t perm[6];                /* Permute / Transpose: PermutationVector */
    int32_t begin[6], end[6], stride[6];        /* StridedSlice; Slice: begin, and the sizes in `end` */
    int32_t begin_mask, end_mask, shrink_axis_mask;
} oracle_move_params;

#ifdef __cplusplus
extern "C" {
#endif
int oracle_move_q(const oracle_move_params* p);
int cpuref_move_q(const oracle_move_params* p);
#ifdef __cplusplus
}
#endif
#endif
