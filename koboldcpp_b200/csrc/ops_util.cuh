// ops_util.cuh -- host / device helpers shared by the op files beside ops.cu: strided tensor descriptors and block reductions.
#pragma once
#include "b200_common.cuh"
#include "../../include/b200_ggml_ops.h"

namespace b200 {
namespace opx {

struct TD {  // device-side tensor descriptor (element counts, byte strides)
    char   *data;
    int64_t ne[4];
    int64_t nb[4];
};
inline TD td(const b200_tensor *t) {
    TD d;
    d.data = (char *)t->data;
    for (int i = 0; i < 4; i++) { d.ne[i] = t->ne[i]; d.nb[i] = (int64_t)t->nb[i]; }
    return d;
}
inline int64_t nelements(const b200_tensor *t) { return t->ne[0] * t->ne[1] * t->ne[2] * t->ne[3]; }
inline int64_t nrows(const b200_tensor *t) { return t->ne[1] * t->ne[2] * t->ne[3]; }
inline bool same_shape(const b200_tensor *a, const b200_tensor *b) {
    return a->ne[0] == b->ne[0] && a->ne[1] == b->ne[1] && a->ne[2] == b->ne[2] && a->ne[3] == b->ne[3];
}
__device__ __forceinline__ char *row_ptr(const TD &t, int64_t r) {
    const int64_t i1 = r % t.ne[1], i2 = (r / t.ne[1]) % t.ne[2], i3 = r / (t.ne[1] * t.ne[2]);
    return t.data + i1 * t.nb[1] + i2 * t.nb[2] + i3 * t.nb[3];
}
// sum over the block; every thread gets the result; sh: 32 floats
__device__ __forceinline__ float block_sum(float v, float *sh) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (nw == 1) return v;
    __syncthreads();
    if (l == 0) sh[w] = v;
    __syncthreads();
    v = l < nw ? sh[l] : 0.f;
    return warp_sum(v);
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

}  // namespace opx
}  // namespace b200

#define OPX_REQUIRE(cond, code, ...)              \
    do {                                          \
        if (!(cond)) {                            \
            b200::set_error(__VA_ARGS__);         \
            return code;                          \
        }                                         \
    } while (0)
