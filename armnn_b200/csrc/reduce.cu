// Reduce (Sum, Max, Mean, Min, Prod over any set of dimensions), the reference's arithmetic: an fp32 accumulator per
// output element that takes the decoded input elements in the order of the flat input index
// (src/backends/reference/workloads/Reduce.cpp:63-175).  One thread per output element walks its reduced elements in
// that order, so Sum / Mean / Prod round exactly as the reference's do; neighbouring threads are neighbouring outputs
// (coalesced whenever the innermost dimension is kept).
#include <cfloat>
#include "common.cuh"

namespace b200k {

struct ReduceArgs {
    QView x, y;
    int nk, nr;                     // kept / reduced dimensions
    int kshape[6], rshape[6];
    long long kstride[6], rstride[6];   // input strides of the kept / reduced dimensions (elements)
    long long outputs, reduced;
    int op;
};

__global__ void __launch_bounds__(128) reduce_kernel(const ReduceArgs a)
{
    pdl_enter();
    const long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (o >= a.outputs) return;
    long long rest = o, base = 0;
    for (int k = a.nk - 1; k >= 0; --k) { base += (rest % a.kshape[k]) * a.kstride[k]; rest /= a.kshape[k]; }
    float acc = (a.op == 0 || a.op == 2) ? 0.f : (a.op == 4 ? 1.f : (a.op == 1 ? -FLT_MAX : FLT_MAX));
    int idx[6] = {0, 0, 0, 0, 0, 0};
    long long off = base;
    for (long long r = 0; r < a.reduced; ++r) {
        const float v = a.x.get(off);
        if (a.op == 0 || a.op == 2) acc = __fadd_rn(acc, v);
        else if (a.op == 4)         acc = __fmul_rn(acc, v);
        else if (a.op == 1)         { if (v > acc) acc = v; }
        else                        { if (v < acc) acc = v; }
        // next reduced index, innermost reduced dimension fastest (increasing flat input index)
        for (int k = a.nr - 1; k >= 0; --k) {
            off += a.rstride[k];
            if (++idx[k] < a.rshape[k]) break;
            off -= a.rstride[k] * a.rshape[k];
            idx[k] = 0;
        }
    }
    if (a.op == 2) acc = __fdiv_rn(acc, (float)a.reduced);
    a.y.set(o, acc);
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_reduce_q(const b200k_reduce_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "reduce_q: null params");
    B200K_REQUIRE(p->x.data && p->y.data, B200K_E_INVALID, "reduce_q: null tensor pointer");
    B200K_REQUIRE(p->rank >= 1 && p->rank <= 6, B200K_E_UNSUPPORTED, "reduce_q: rank %d not in [1, 6]", p->rank);
    B200K_REQUIRE(p->op >= 0 && p->op <= 4, B200K_E_INVALID, "reduce_q: operation %d not in [0, 4]", p->op);
    B200K_REQUIRE(p->x.dtype != B200K_S32 && p->y.dtype != B200K_S32, B200K_E_UNSUPPORTED, "reduce_q: Signed32 not supported");
    B200K_REQUIRE((p->axis_mask >> p->rank) == 0 && p->axis_mask >= 0, B200K_E_INVALID, "reduce_q: axis outside the tensor's rank");
    const int mask = p->axis_mask ? p->axis_mask : (1 << p->rank) - 1;
    ReduceArgs a;
    memset(&a, 0, sizeof(a));
    a.x = make_view(p->x); a.y = make_view(p->y);
    a.op = p->op;
    a.outputs = 1; a.reduced = 1;
    long long stride[6], st = 1;
    for (int d = p->rank - 1; d >= 0; --d) {
        B200K_REQUIRE(p->shape[d] > 0, B200K_E_INVALID, "reduce_q: empty dimension");
        stride[d] = st; st *= p->shape[d];
    }
    for (int d = 0; d < p->rank; ++d) {
        if (mask & (1 << d)) { a.rshape[a.nr] = p->shape[d]; a.rstride[a.nr] = stride[d]; ++a.nr; a.reduced *= p->shape[d]; }
        else                 { a.kshape[a.nk] = p->shape[d]; a.kstride[a.nk] = stride[d]; ++a.nk; a.outputs *= p->shape[d]; }
    }
    launch_pdl(reduce_kernel, dim3(div_up(a.outputs, 128)), dim3(128), 0, (cudaStream_t)stream, a);
    return check_launch("reduce_kernel");
}
