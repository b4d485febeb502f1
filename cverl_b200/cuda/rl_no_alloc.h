// An entry point of the RL kernel library that allocates nothing.
//
// This has no counterpart in the reference: it exists for callers that must not allocate device
// memory at the point of the call.  Two kinds of caller are meant.  One runs inside a region where
// an allocation would either fail or silently change behaviour: a caller that has pinned the
// device's memory budget up front (a rollout engine that gave all remaining memory to its KV
// cache), where a late allocation can run out of memory at a random step.  The other sits on a
// latency path between two kernels of a step, where an allocator call may take a lock, touch the
// driver or synchronise, and where the plain entry point would force the caller to own and thread
// through a scratch pointer just for this one op.
//
// cvb_grpo_advantage_static computes exactly what cvb_grpo_advantage computes (per-row outcome
// score, group mean / std normalisation, broadcast over the masked response tokens), but its
// per-row scratch lives in a fixed array in the library's device image instead of a buffer of
// the caller's.  Limits and rules:
//
//  * rows <= CVB_GRPO_STATIC_MAX_ROWS.  A larger batch is rejected with
//    CVB_ERR_STATIC_SCRATCH_LIMIT (and one line on stderr) before anything is launched.
//  * The first call on a device looks up the array's device address, once, with that device
//    current.  That call is set-up work: make it before any stream capture begins.
//  * Every call on a device shares the one array.  Nothing in it has to start at zero: each call
//    writes every word it later reads.  Calls that may overlap in time on one device (different
//    streams, different host threads) race on it; order them on one stream or with events.
#pragma once

#define CVB_GRPO_STATIC_MAX_ROWS 16384          // 2 floats of scratch per row: 128 KB per device
#define CVB_ERR_STATIC_SCRATCH_LIMIT (-1001)    // rows beyond the fixed scratch
#define CVB_ERR_STATIC_SCRATCH_SETUP (-1002)    // the address look-up failed (the CUDA error is printed)

#ifdef __cplusplus
extern "C" {
#endif

// rewards, mask, adv, ret: fp32 [rows, cols] on the current device; gid: int64 [rows]; ret may be null.
// Returns 0, a CVB_ERR_STATIC_* code, or the CUDA error of a failed launch.
int cvb_grpo_advantage_static(const float* rewards, const float* mask, const long long* gid, float eps,
                              int norm_by_std, float* adv, float* ret, long long rows, int cols, void* stream);

#ifdef __cplusplus
}
#endif
