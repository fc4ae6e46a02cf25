// One QLstm step, reproducing RefQLstmWorkload::Execute operation by operation
// (src/backends/reference/workloads/RefQLstmWorkload.cpp:46-541, LstmUtils.cpp:16-256 of the Arm NN tree).
//
// CpuRef keeps the gate pre-activations in int16 buffers and re-quantises them after EVERY
// multiply-accumulate of the mat-vec products (LstmUtils.cpp:87-111), so a gate value is the end of a
// K-long chain  acc <- Q16(deq(acc) + deq(w) * deq(x))  whose result depends on every intermediate rounding
// and saturation.  An int32 dot product followed by one requantisation is a different function, so the
// kernel evaluates the chains themselves: one chain per (gate, unit) of a batch row, all chains of a row
// in one CTA, 2 chains per thread for instruction-level parallelism, and the GPU hides the chain latency
// by running every (row, gate, unit) chain concurrently.  This is latency/issue-bound fp32 work: no
// tensor cores.  The int16 accumulator is carried as an integer-valued float (the clamp keeps it in
// [-32768, 32767], where float is exact), which removes two conversions per step without changing a bit.
//
// One CTA handles one batch row through the whole step: mat-vecs -> (peephole) -> layer norm ->
// activations -> cell update -> output gate -> hidden state -> projection -> outputs.  Layer-norm sums
// are accumulated by a single thread per gate in index order because CpuRef's fp32 sums are sequential.
#include "common.cuh"

namespace b200k {

constexpr int QL_THREADS = 1024;

__device__ __forceinline__ float q16f(float v, float scale)          // Quantize<int16_t>, offset 0, as float
{
    return fminf(fmaxf(roundf(__fdiv_rn(v, scale)), -32768.f), 32767.f);
}
__device__ __forceinline__ float q16zf(float v, float scale, float zp)
{
    return fminf(fmaxf(__fadd_rn(zp, roundf(__fdiv_rn(v, scale))), -32768.f), 32767.f);
}

// round_half_away(fl(v / scale)) without the division unit, for the long chains: with inv = RN(1 / scale)
// (__frcp_rn), p = fl(v * inv) and q = fma(fma(-p, scale, v), inv, p) is the correctly rounded quotient (Markstein);
// q is rounded with the 1.5 * 2^23 constant (halves to even), and only when q is an exact half or too large for the
// constant does roundf decide.
__device__ __forceinline__ float round_div_fast(float v, float scale, float inv)
{
    const float p = __fmul_rn(v, inv);
    const float q = __fmaf_rn(__fmaf_rn(-p, scale, v), inv, p);
    float n = __fsub_rn(__fadd_rn(q, 12582912.0f), 12582912.0f);
    if (fabsf(__fsub_rn(q, n)) >= 0.5f) n = roundf(q);
    return n;
}
__device__ __forceinline__ float q16f_fast(float v, float scale, float inv)
{
    return fminf(fmaxf(round_div_fast(v, scale, inv), -32768.f), 32767.f);
}
__device__ __forceinline__ float q16zf_fast(float v, float scale, float inv, float zp)
{
    return fminf(fmaxf(__fadd_rn(zp, round_div_fast(v, scale, inv)), -32768.f), 32767.f);
}

struct QlArgs {
    b200k_qlstm_params p;
    int cifg, peephole, ln, proj;
};

// acc <- chain over k of Q16(acc*sG + (w[k]*sw) * v[k]) for two independent chains (A and B), both evaluated by
// packed two-wide fp32 instructions (the chains of a row keep the schedulers' issue slots busy, so halving the
// instruction count is what counts).  v2 holds every value twice, as (x, x) pairs.  Products that the reference
// rounds before adding are formed as fma2(a, b, 0): a packed multiply feeding a packed add would be contracted.
// Quantize to int16: Markstein's correctly rounded quotient, the 1.5 * 2^23 rounding constant, and roundf for the
// exact halves it rounds to even where the reference rounds away from zero (see round_div_fast).
template <bool VEC>
__device__ __forceinline__ void chain2(float& accA, float& accB, const int8_t* wA, const int8_t* wB, float swA, float swB,
                                        const float2* v2, int K, float sGA, float sGB, bool hasB)
{
    const float iGA = __frcp_rn(sGA), iGB = __frcp_rn(sGB);
    const f32x2 sG2 = pack2(sGA, sGB), nsG2 = pack2(-sGA, -sGB), iG2 = pack2(iGA, iGB), sw2 = pack2(swA, swB);
    const f32x2 zero2 = pack2(0.f, 0.f), magic2 = pack2(12582912.0f, 12582912.0f);
    f32x2 acc2 = pack2(accA, accB);
    auto step = [&](float wa, float wb, int k) {
        const float2 xx = v2[k];
        const f32x2 t2 = fma2(fma2(pack2(wa, wb), sw2, zero2), pack2(xx.x, xx.y), zero2);    // fl(fl(w * sw) * x)
        const f32x2 a2 = add2(fma2(acc2, sG2, zero2), t2);                                    // fl(fl(acc * sG) + t)
        const f32x2 p2 = mul2(a2, iG2);
        const f32x2 q2 = fma2(fma2(p2, nsG2, a2), iG2, p2);                                   // RN(a / sG)
        const f32x2 n2 = sub2(add2(q2, magic2), magic2);
        float qa, qb, na, nb;
        unpack2(q2, qa, qb); unpack2(n2, na, nb);
        if (fabsf(__fsub_rn(qa, na)) >= 0.5f) na = roundf(qa);
        if (fabsf(__fsub_rn(qb, nb)) >= 0.5f) nb = roundf(qb);
        acc2 = pack2(fminf(fmaxf(na, -32768.f), 32767.f), fminf(fmaxf(nb, -32768.f), 32767.f));
    };
    if (VEC) {
        for (int k0 = 0; k0 < K; k0 += 16) {
            int8_t ra[16], rb[16];
            *(uint4*)ra = *(const uint4*)(wA + k0);
            if (hasB) *(uint4*)rb = *(const uint4*)(wB + k0);
            else      *(uint4*)rb = make_uint4(0, 0, 0, 0);
            #pragma unroll
            for (int j = 0; j < 16; ++j) step((float)ra[j], (float)rb[j], k0 + j);
        }
    } else {
        for (int k = 0; k < K; ++k) step((float)wA[k], hasB ? (float)wB[k] : 0.f, k);
    }
    unpack2(acc2, accA, accB);
}

template <bool VEC_I, bool VEC_O>
__global__ void __launch_bounds__(QL_THREADS) qlstm_step_kernel(const QlArgs a)
{
    pdl_enter();
    const b200k_qlstm_params& p = a.p;
    const int I = p.input_size, U = p.num_units, O = p.output_size;
    const int b = blockIdx.x, tid = threadIdx.x;
    extern __shared__ float sm[];
    float2* xf = (float2*)sm;       // [I]   dequantised input row, every value twice (for the two-wide chains)
    float2* hf = xf + I;            // [O]   dequantised previous output state, likewise
    float* gate = (float*)(hf + O); // [4][U] int16 gate buffers as integer-valued floats (i, f, c, o)
    float* cell = gate + 4 * U;     // [U]   new cell state (integer-valued)
    float* hid = cell + U;          // [U]   dequantised hidden state
    float* stat = hid + U;          // [4][2] mean, 1/stddev per gate

    for (int k = tid; k < I; k += QL_THREADS) {
        const float v = dequantize_dev(p.input[(long long)b * I + k], p.input_scale, p.input_zp);
        xf[k] = make_float2(v, v);
    }
    for (int k = tid; k < O; k += QL_THREADS) {
        const float v = dequantize_dev(p.output_state_in[(long long)b * O + k], p.output_state_scale, p.output_state_zp);
        hf[k] = make_float2(v, v);
    }
    __syncthreads();

    const int8_t* wi[4] = {p.w_i2i, p.w_i2f, p.w_i2c, p.w_i2o};
    const int8_t* wr[4] = {p.w_r2i, p.w_r2f, p.w_r2c, p.w_r2o};
    const float si[4] = {p.s_i2i, p.s_i2f, p.s_i2c, p.s_i2o};
    const float sr[4] = {p.s_r2i, p.s_r2f, p.s_r2c, p.s_r2o};
    const float sint[4] = {p.input_intermediate_scale, p.forget_intermediate_scale, p.cell_intermediate_scale,
                           p.output_intermediate_scale};
    const int g0 = a.cifg ? 1 : 0;
    const int nchains = (4 - g0) * U;

    // ---- mat-vec chains: input weights first, then recurrent weights, continuing the same accumulator
    for (int c0 = tid; c0 < nchains; c0 += 2 * QL_THREADS) {
        const int cA = c0, cB = c0 + QL_THREADS;
        const bool hasB = cB < nchains;
        const int gA = g0 + cA / U, uA = cA % U;
        const int gB = hasB ? g0 + cB / U : gA, uB = hasB ? cB % U : uA;
        float accA = 0.f, accB = 0.f;
        chain2<VEC_I>(accA, accB, wi[gA] + (long long)uA * I, wi[gB] + (long long)uB * I, si[gA], si[gB], xf, I,
                      sint[gA], sint[gB], hasB);
        chain2<VEC_O>(accA, accB, wr[gA] + (long long)uA * O, wr[gB] + (long long)uB * O, sr[gA], sr[gB], hf, O,
                      sint[gA], sint[gB], hasB);
        gate[gA * U + uA] = accA;
        if (hasB) gate[gB * U + uB] = accB;
    }
    __syncthreads();

    const float sc = p.cell_state_scale;
    const int16_t* peep[4] = {p.w_c2i, p.w_c2f, nullptr, p.w_c2o};
    const float speep[4] = {p.s_c2i, p.s_c2f, 0.f, p.s_c2o};
    const int16_t* lnw[4] = {p.ln_i, p.ln_f, p.ln_c, p.ln_o};
    const float slnw[4] = {p.s_lni, p.s_lnf, p.s_lnc, p.s_lno};
    const int32_t* gbias[4] = {p.b_i, p.b_f, p.b_c, p.b_o};
    const float sgb[4] = {p.s_bi, p.s_bf, p.s_bc, p.s_bo};

    // Post-processing of gates [gfirst, glast]: peephole, layer norm, activation.  `cellsrc` is the cell
    // state the peephole reads (old state for i and f, new state for o), as integer-valued floats.
    auto gate_post = [&](int gfirst, int glast, const int16_t* cell_in_global, const float* cell_smem) {
        if (a.peephole) {
            for (int t = tid; t < (glast - gfirst + 1) * U; t += QL_THREADS) {
                const int g = gfirst + t / U, u = t % U;
                if (!peep[g]) continue;
                const float cv = cell_smem ? cell_smem[u] : (float)cell_in_global[(long long)b * U + u];
                const float pr = __fmul_rn(__fmul_rn((float)peep[g][u], speep[g]), __fmul_rn(cv, sc));
                gate[g * U + u] = q16f(__fadd_rn(__fmul_rn(gate[g * U + u], sint[g]), pr), sint[g]);
            }
            __syncthreads();
        }
        if (a.ln) {
            // sequential sums, one thread (in its own warp) per gate: LstmUtils.cpp:46-53
            const int w = tid >> 5;
            if ((tid & 31) == 0 && w <= glast - gfirst) {
                const int g = gfirst + w;
                float sum = 0.f, sum_sq = 0.f;
                for (int i = 0; i < U; ++i) {
                    const float v = __fmul_rn(gate[g * U + i], sint[g]);
                    sum = __fadd_rn(sum, v);
                    sum_sq = __fadd_rn(sum_sq, __fmul_rn(v, v));
                }
                const float fu = (float)U;
                const float mean = __fdiv_rn(sum, fu);
                const float variance = __fsub_rn(__fdiv_rn(sum_sq, fu), __fmul_rn(mean, mean));
                const float sd = variance == 0.f ? __fsqrt_rn(1e-8f) : __fsqrt_rn(variance);
                stat[g * 2] = mean;
                stat[g * 2 + 1] = __fdiv_rn(1.0f, sd);
            }
            __syncthreads();
        }
        for (int t = tid; t < (glast - gfirst + 1) * U; t += QL_THREADS) {
            const int g = gfirst + t / U, u = t % U;
            float q = gate[g * U + u];
            float s = sint[g];
            if (a.ln) {
                const float sln = __fmul_rn(__fmul_rn(p.input_scale, slnw[g]), 1024.f);
                q = q16f(__fmul_rn(__fsub_rn(__fmul_rn(q, s), stat[g * 2]), stat[g * 2 + 1]), sln);       // normalise
                q = q16f(__fmul_rn(__fmul_rn((float)lnw[g][u], slnw[g]), __fmul_rn(q, sln)), sln);           // * weight
                q = q16f(__fadd_rn(__fmul_rn(q, sln), __fmul_rn(__int2float_rn(gbias[g][u]), sgb[g])), 1.f / 4096);  // + bias
                s = 1.f / 4096;
            }
            const float v = __fmul_rn(q, s);
            const float r = g == 2 ? tanhf(v) : __fdiv_rn(1.f, __fadd_rn(1.f, expf(-v)));
            gate[g * U + u] = q16f(r, sc);
        }
        __syncthreads();
    };

    gate_post(g0, 2, p.cell_state_in, nullptr);

    // ---- cell state: c = Q(f * c_in); c = Q(c + g * i)  (or g * Q(1 - f) with CIFG); clip
    for (int u = tid; u < U; u += QL_THREADS) {
        const float cin = __fmul_rn((float)p.cell_state_in[(long long)b * U + u], sc);
        const float f = gate[1 * U + u];
        float c = q16f(__fmul_rn(__fmul_rn(f, sc), cin), sc);
        const float ig = a.cifg ? q16f(__fsub_rn(1.0f, __fmul_rn(f, sc)), sc) : gate[0 * U + u];
        c = q16f(__fadd_rn(__fmul_rn(c, sc), __fmul_rn(__fmul_rn(gate[2 * U + u], sc), __fmul_rn(ig, sc))), sc);
        if (p.cell_clip > 0.0f) {
            const float fv = __fmul_rn(c, sc);
            float r = (p.cell_clip < fv) ? p.cell_clip : fv;
            r = (-p.cell_clip > r) ? -p.cell_clip : r;
            c = q16f(r, sc);
        }
        cell[u] = c;
        p.cell_state_out[(long long)b * U + u] = (int16_t)c;
    }
    __syncthreads();

    gate_post(3, 3, nullptr, cell);

    // ---- hidden = Q8(o * Q16(tanh(c)))
    const float hzp = (float)p.hidden_state_zp;
    for (int u = tid; u < U; u += QL_THREADS) {
        const float t = q16f(tanhf(__fmul_rn(cell[u], sc)), sc);
        const float hv = __fmul_rn(__fmul_rn(gate[3 * U + u], sc), __fmul_rn(t, sc));
        const float hq = fminf(fmaxf(__fadd_rn(hzp, roundf(__fdiv_rn(hv, p.hidden_state_scale))), -128.f), 127.f);
        hid[u] = __fmul_rn(__fsub_rn(hq, hzp), p.hidden_state_scale);      // dequantised hidden state
    }
    __syncthreads();

    // ---- projection (int16 accumulator at the OUTPUT's scale and offset) and outputs
    const float so = p.output_scale, zo = (float)p.output_zp, iso = __frcp_rn(p.output_scale);
    for (int j = tid; j < O; j += QL_THREADS) {
        float out8;
        if (a.proj) {
            float acc = 0.f;                                   // int16 buffer starts as raw zeros
            if (p.b_proj) acc = q16zf(__fmul_rn(__int2float_rn(p.b_proj[j]), p.s_bproj), so, zo);
            const int8_t* w = p.w_proj + (long long)j * U;
            for (int k = 0; k < U; ++k) {
                const float d = __fmul_rn(__fsub_rn(acc, zo), so);
                acc = q16zf_fast(__fadd_rn(d, __fmul_rn(__fmul_rn((float)w[k], p.s_proj), hid[k])), so, iso, zo);
            }
            out8 = fminf(fmaxf(__fadd_rn(zo, roundf(__fdiv_rn(__fmul_rn(__fsub_rn(acc, zo), so), so))), -128.f), 127.f);
            if (p.projection_clip > 0.0f) {
                const float fv = __fmul_rn(__fsub_rn(out8, zo), so);
                float r = (p.projection_clip < fv) ? p.projection_clip : fv;
                r = (-p.projection_clip > r) ? -p.projection_clip : r;
                out8 = fminf(fmaxf(__fadd_rn(zo, roundf(__fdiv_rn(r, so))), -128.f), 127.f);
            }
        } else {
            out8 = fminf(fmaxf(__fadd_rn(zo, roundf(__fdiv_rn(hid[j], so))), -128.f), 127.f);
        }
        p.output[(long long)b * O + j] = (int8_t)out8;
        const float ov = __fmul_rn(__fsub_rn(out8, zo), so);
        const float hs = fminf(fmaxf(__fadd_rn((float)p.output_state_zp, roundf(__fdiv_rn(ov, p.output_state_scale))), -128.f), 127.f);
        p.output_state_out[(long long)b * O + j] = (int8_t)hs;
    }
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_qlstm_step(const b200k_qlstm_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "qlstm_step: null params");
    B200K_REQUIRE(p->batch > 0 && p->input_size > 0 && p->num_units > 0 && p->output_size > 0, B200K_E_INVALID,
                  "qlstm_step: bad shape");
    B200K_REQUIRE(p->input && p->output_state_in && p->cell_state_in && p->output_state_out && p->cell_state_out &&
                  p->output, B200K_E_INVALID, "qlstm_step: null state/input/output pointer");
    B200K_REQUIRE(p->w_i2f && p->w_i2c && p->w_i2o && p->w_r2f && p->w_r2c && p->w_r2o, B200K_E_INVALID,
                  "qlstm_step: missing mandatory weights");
    QlArgs a;
    a.p = *p;
    a.cifg = p->w_i2i == nullptr;
    a.peephole = p->w_c2f != nullptr;
    a.ln = p->ln_f != nullptr;
    a.proj = p->w_proj != nullptr;
    B200K_REQUIRE(a.cifg || p->w_r2i, B200K_E_INVALID, "qlstm_step: input-to-input weights without recurrent-to-input weights");
    B200K_REQUIRE(!a.peephole || (p->w_c2o && (a.cifg || p->w_c2i)), B200K_E_INVALID, "qlstm_step: incomplete peephole weights");
    B200K_REQUIRE(!a.ln || (p->ln_c && p->ln_o && (a.cifg || p->ln_i) && p->b_f && p->b_c && p->b_o && (a.cifg || p->b_i)),
                  B200K_E_INVALID, "qlstm_step: layer norm needs all layer-norm weights and gate biases");
    B200K_REQUIRE(a.proj || p->num_units == p->output_size, B200K_E_INVALID,
                  "qlstm_step: without projection the output size must equal the number of units");
    const size_t smem = sizeof(float) * (2 * ((size_t)p->input_size + p->output_size) + 6 * (size_t)p->num_units + 8);
    B200K_REQUIRE(smem <= 200 * 1024, B200K_E_TOOBIG, "qlstm_step: layer too large for the shared-memory resident kernel");
    const bool vi = (p->input_size % 16) == 0 &&
                    ((((uintptr_t)p->w_i2i | (uintptr_t)p->w_i2f | (uintptr_t)p->w_i2c | (uintptr_t)p->w_i2o) & 15) == 0);
    const bool vo = (p->output_size % 16) == 0 &&
                    ((((uintptr_t)p->w_r2i | (uintptr_t)p->w_r2f | (uintptr_t)p->w_r2c | (uintptr_t)p->w_r2o) & 15) == 0);
    cudaStream_t s = (cudaStream_t)stream;
    auto launch = [&](auto kern) -> int {
        if (smem > 48 * 1024) B200K_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        launch_pdl(kern, dim3((unsigned)p->batch), dim3(QL_THREADS), smem, s, a);
        return check_launch("qlstm_step_kernel");
    };
    if (vi && vo)  return launch(qlstm_step_kernel<true, true>);
    if (!vi && vo) return launch(qlstm_step_kernel<false, true>);
    if (vi && !vo) return launch(qlstm_step_kernel<true, false>);
    return launch(qlstm_step_kernel<false, false>);
}
