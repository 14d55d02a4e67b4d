// Builds the reference's OWN OpenCL C source of the counter kernels as host C++.
// TEST INFRASTRUCTURE ONLY: it validates oracle/counter_oracle.cpp and generates the
// golden vectors in tests/golden/.  Nothing shipped links or loads it.
//
// The reference file is included by path at build time (macro MOTIFCL_COUNTER_CL, set by
// oracle/Makefile to <reference>/kernels/compact_counter.cl); no reference source is
// copied into this repository.  The shim supplies the handful of OpenCL C names the
// file uses:
//   * address-space and kernel qualifiers expand to nothing (__local becomes `static`,
//     so a work-group's shared arrays are one array shared by the emulating threads);
//   * work-item ids come from thread-local variables set by the launchers below;
//   * barrier() is a real std::barrier across the work-group's threads, so the two
//     row-statistics kernels (which use __local memory and barriers) execute with true
//     64-lane semantics: 64 host threads per work-group, one work-group at a time;
//   * clamp/fmax/floor/trunc/sqrt resolve to the float overloads of <cmath>.
// Build flags (-ffp-contract=off, no fast-math) make '/' and sqrt correctly rounded and
// forbid FMA contraction; that choice defines "the reference result" on a CPU.

#include <barrier>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <thread>
#include <vector>

namespace refcl {

typedef unsigned char uchar;
typedef unsigned int uint;

struct WorkItem {
    int global_id = 0, local_id = 0, group_id = 0, local_size = 1;
    std::barrier<>* bar = nullptr;
};
thread_local WorkItem g_wi;

inline int get_global_id(int) { return g_wi.global_id; }
inline int get_local_id(int) { return g_wi.local_id; }
inline int get_group_id(int) { return g_wi.group_id; }
inline int get_local_size(int) { return g_wi.local_size; }
inline void barrier(int) {
    if (g_wi.bar) g_wi.bar->arrive_and_wait();
}
inline float clamp(float x, float lo, float hi) { return std::fmin(std::fmax(x, lo), hi); }
using std::floor;
using std::fmax;
using std::sqrt;
using std::trunc;

#define __kernel
#define __global
#define __local static
#define CLK_LOCAL_MEM_FENCE 0

#include MOTIFCL_COUNTER_CL

#undef __kernel
#undef __global
#undef __local

// Run `body` once per work-item of a 1-D range with no barriers: serial loop.
template <class F>
void launch_flat(int global, F body) {
    for (int gid = 0; gid < global; ++gid) {
        g_wi = WorkItem{gid, 0, 0, 1, nullptr};
        body();
    }
}

// Run `body` for `groups` work-groups of `lsz` work-items with working barriers.  The
// threads of a group are real threads; groups run one after another because the
// kernel's __local arrays are function-scope statics.
template <class F>
void launch_groups(int groups, int lsz, F body) {
    for (int grp = 0; grp < groups; ++grp) {
        std::barrier<> bar(lsz);
        std::vector<std::thread> th;
        th.reserve(lsz);
        for (int lid = 0; lid < lsz; ++lid)
            th.emplace_back([&, lid] {
                g_wi = WorkItem{grp * lsz + lid, lid, grp, lsz, &bar};
                body();
            });
        for (auto& t : th) t.join();
    }
}

}  // namespace refcl

extern "C" {

// kernels/compact_counter.cl:39-55
void ref_decode_weight(const uint8_t* state, const float* scale, float* w, int C, int in_features,
                       int out_features) {
    const int n_groups = out_features * (in_features / 4);
    refcl::launch_flat(n_groups, [&] {
        refcl::decode_counter_state_weight_f32(state, scale, w, C, in_features, n_groups);
    });
}

// Dense update exactly as src/nn/compact_counter.cpp:113-156 launches it:
// counter_row_stats_f32 (one 64-wide group per row), counter_apply_update_f32 (one item
// per packed group), then scale <- scale_new.
void ref_update_dense(uint8_t* state, float* scale, float* v, const float* grad_w, int C,
                      int in_features, int out_features, float lr, float lr_scale, float rms_beta,
                      float rms_eps, uint32_t seed) {
    std::vector<float> scale_new(out_features), denom(out_features);
    refcl::launch_groups(out_features, 64, [&] {
        refcl::counter_row_stats_f32(state, scale, v, grad_w, scale_new.data(), denom.data(), C,
                                     in_features, out_features, lr_scale, rms_beta, rms_eps);
    });
    const int n_groups = out_features * (in_features / 4);
    refcl::launch_flat(n_groups, [&] {
        refcl::counter_apply_update_f32(state, scale, scale_new.data(), denom.data(), grad_w, C,
                                        in_features, n_groups, lr, seed);
    });
    std::memcpy(scale, scale_new.data(), sizeof(float) * out_features);
}

// Memory-native update exactly as src/nn/compact_counter.cpp:158-231 launches it.
void ref_update_fused(uint8_t* state, float* scale, float* v, const float* grad_out, const float* x,
                      int C, int in_features, int out_features, int N, float lr, float lr_scale,
                      float rms_beta, float rms_eps, uint32_t seed) {
    std::vector<float> scale_new(out_features), denom(out_features);
    refcl::launch_groups(out_features, 64, [&] {
        refcl::counter_row_stats_fused_f32(state, scale, v, grad_out, x, scale_new.data(),
                                           denom.data(), C, in_features, out_features, N, lr_scale,
                                           rms_beta, rms_eps);
    });
    const int n_groups = out_features * (in_features / 4);
    refcl::launch_flat(n_groups, [&] {
        refcl::counter_apply_update_fused_f32(state, scale, scale_new.data(), denom.data(), grad_out,
                                              x, C, in_features, out_features, N, n_groups, lr, seed);
    });
    std::memcpy(scale, scale_new.data(), sizeof(float) * out_features);
}

// kernels/compact_counter.cl:248-269
void ref_backward_input(const float* grad_out, const uint8_t* state, const float* scale,
                        float* grad_x, int C, int in_features, int out_features, int N) {
    refcl::launch_flat(N * in_features, [&] {
        refcl::counter_backward_input_f32(grad_out, state, scale, grad_x, C, in_features,
                                          out_features, N);
    });
}

}  // extern "C"
