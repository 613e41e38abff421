// Host interface of the tcgen05 / TMEM / TMA kernel family (KSMM_ALGO_TC).
#pragma once

#include "common.cuh"

namespace ksmm {

int tc_num_configs();
// true if configuration `config` of the family can run problem `p`
// (element types, layout, TMA alignment rules).  With check_pointers the
// base addresses are checked as well.
bool tc_config_supported(const Problem& p, int config, bool check_pointers);
// heuristic default configuration, or -1 if the family cannot run `p`
int tc_default_config(const Problem& p);
int tc_launch(const Problem& p, int config, cudaStream_t stream);
// true if the kernel tc_launch runs for `p` adds p.residual in its epilogue
bool tc_fuses_residual(const Problem& p);
// true if `p` (with out_regroup_c / out_regroup_d set) can store its output regrouped by the
// blocks of the next factor of a chain
bool tc_can_regroup_output(const Problem& p);
// Synchronises `stream` and reports a device-side timeout recorded by any
// earlier launch of this family on the current device (then clears it).
int tc_check_device(cudaStream_t stream);
// Launches one warp whose bounded wait (limit in SM cycles) is certain to run out; the device
// status word then holds `code`.  Test hook for the timeout path.
int tc_wait_probe(long long limit_cycles, int code, cudaStream_t stream);

// batch-first factors with d = 2 or 4 (tc_bsfirst_d.cu); a single configuration
bool tc_bsfirst_d_supported(const Problem& p, bool check_pointers);
int tc_bsfirst_d_launch(const Problem& p, cudaStream_t stream);

// batch-first factors with d a multiple of 8 (tc_bsfirst_g.cu): groups of eight blocks per CTA
bool tc_bsfirst_g_supported(const Problem& p, bool check_pointers);
int tc_bsfirst_g_launch(const Problem& p, cudaStream_t stream);

// batch-first factors with d = 2 or 4 through a regrouping pass and a kernel without the
// transposer stage (tc_bsfirst_dp.cu); configuration 1 of such problems
bool tc_bsfirst_dp_supported(const Problem& p, bool check_pointers);
int tc_bsfirst_dp_launch(const Problem& p, cudaStream_t stream);
// bytes of layout scratch that launch needs (0 when the input is regrouped already)
size_t tc_bsfirst_dp_scratch_bytes(const Problem& p);

// fp32 factors as three tf32 products per term (tc_f32x3.cu); configuration 0 picks the j tile by
// a cost rule, 1..3 force 128, 96 and 64 columns (what the tuner compares)
bool tc_f32x3_supported(const Problem& p, bool check_pointers);
int tc_f32x3_launch(const Problem& p, int config, cudaStream_t stream);

}  // namespace ksmm
