// Instantiation list for compiling the reference's own kernels as a checker (oracle/_ref):
// the launch shapes the reference tuned for its newest GPU (scripts/optima-fixed-max_slowdown.csv:
// bits-prefetch block 256 / batch 13; fused-cache 8,4,2 with block-query-dim 1, dim-mult 1) plus
// batch 16 and dim-mult 2.  Shadows the reference's definitions_minimal.hpp on the include path.
#ifndef TOPK_SINGLEPASS_DETAIL_DEFINITIONS_MINIMAL_HPP_
#define TOPK_SINGLEPASS_DETAIL_DEFINITIONS_MINIMAL_HPP_

#define TOPK_SINGLEPASS_BITS_BATCH_SIZES 13, 16
#define TOPK_SINGLEPASS_BITS_BLOCK_SIZES 256

#define TOPK_SINGLEPASS_FC_DIM_REGS 2
#define TOPK_SINGLEPASS_FC_DIM_MULTS 1, 2
#define TOPK_SINGLEPASS_FC_QUERY_REGS 8
#define TOPK_SINGLEPASS_FC_DB_REGS 4
#define TOPK_SINGLEPASS_FC_BLOCK_QUERY_DIMS 1, 2, 4

#endif
