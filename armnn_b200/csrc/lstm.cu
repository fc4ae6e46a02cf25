// One Float32 LSTM step, operation by operation as armnn::LstmImpl performs it
// (src/backends/reference/workloads/Lstm.cpp:14-259, LstmUtils.cpp of the Arm NN tree): the Lstm layer and every time step
// of UnidirectionalSequenceLstm.
//
// The reference accumulates every gate pre-activation term by term in fp32 (bias, then the input weights over the input,
// then the recurrent weights over the previous output, then the peephole term), so a value is the end of a chain of
// rounded additions.  The kernel evaluates those chains as they are: one CTA per batch row, one chain per (gate, unit)
// spread over the CTA's threads, input and previous output staged in shared memory, weights read once from global
// memory.  Layer-normalisation sums are accumulated by one thread per gate in index order, like the reference's.  This
// is latency-bound fp32 work; no tensor cores.
#include "common.cuh"

namespace b200k {

constexpr int LSTM_THREADS = 256;

__device__ __forceinline__ float lstm_act(float in, int fn)          // LstmUtils.cpp:258-297 + Activation.cpp
{
    switch (fn) {
        case 1: return fmaxf(in, 0.f);
        case 3: return fminf(fmaxf(in, 0.f), 6.f);
        case 4: return tanhf(in);
        case 6: return __fdiv_rn(1.f, __fadd_rn(1.f, expf(-in)));
        default: return in;
    }
}

__device__ __forceinline__ float lstm_clip(float v, float limit)     // LstmUtils.cpp:221-227
{
    float r = limit < v ? limit : v;
    return -limit > r ? -limit : r;
}

// pre-activation of units [tid, tid + threads, ...) of one gate: bias (unless layer norm), input terms, recurrent terms, peephole
__device__ void lstm_gate(const b200k_lstm_params& p, const float* sx, const float* sh, const float* wi, const float* wr,
                          const float* peephole, const float* cell, const float* bias, bool ln, float* out)
{
    for (int u = threadIdx.x; u < p.num_units; u += LSTM_THREADS) {
        float acc = ln ? 0.0f : bias[u];
        const float* wrow = wi + (long long)u * p.input_size;
        for (int k = 0; k < p.input_size; ++k) acc = __fadd_rn(acc, __fmul_rn(wrow[k], sx[k]));
        wrow = wr + (long long)u * p.output_size;
        for (int k = 0; k < p.output_size; ++k) acc = __fadd_rn(acc, __fmul_rn(wrow[k], sh[k]));
        if (peephole) acc = __fadd_rn(acc, __fmul_rn(peephole[u], cell[u]));
        out[u] = acc;
    }
}

// MeanStddevNormalization, then the layer-norm weight and the bias (Lstm.cpp:125-131): `stats` = {mean, 1 / stddev}
__device__ void lstm_layer_norm(const b200k_lstm_params& p, float* g, const float* w, const float* bias, float* stats)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.f, sum_sq = 0.f;
        for (int u = 0; u < p.num_units; ++u) { sum = __fadd_rn(sum, g[u]); sum_sq = __fadd_rn(sum_sq, __fmul_rn(g[u], g[u])); }
        const float n = (float)p.num_units;
        const float mean = __fdiv_rn(sum, n);
        const float variance = __fsub_rn(__fdiv_rn(sum_sq, n), __fmul_rn(mean, mean));
        stats[0] = mean;
        stats[1] = __fdiv_rn(1.0f, __fsqrt_rn(variance == 0.f ? p.layer_norm_eps : variance));
    }
    __syncthreads();
    const float mean = stats[0], inv = stats[1];
    for (int u = threadIdx.x; u < p.num_units; u += LSTM_THREADS)
        g[u] = __fadd_rn(__fmul_rn(w[u], __fmul_rn(__fsub_rn(g[u], mean), inv)), bias[u]);
    __syncthreads();
}

__global__ void __launch_bounds__(LSTM_THREADS) lstm_step_kernel(const b200k_lstm_params p)
{
    pdl_enter();
    extern __shared__ float smem[];
    __shared__ float stats[2];
    const int U = p.num_units, O = p.output_size, I = p.input_size;
    float* sx = smem;            // [I]
    float* sh = sx + I;          // [O]
    float* gi = sh + O;          // [U] each
    float* gf = gi + U;
    float* gc = gf + U;
    float* go = gc + U;
    float* cn = go + U;          // the new cell state
    const int b = blockIdx.x;
    const float* x = p.input + b * p.input_stride;
    const float* h = p.output_state_in + (long long)b * O;
    const float* c_in = p.cell_state_in + (long long)b * U;
    float* c_out = p.cell_state_out + (long long)b * U;
    float* out = p.output + b * p.output_stride;
    const bool cifg = p.w_i2i == nullptr, ln = p.ln_f != nullptr;
    for (int k = threadIdx.x; k < I; k += LSTM_THREADS) sx[k] = x[k];
    for (int k = threadIdx.x; k < O; k += LSTM_THREADS) sh[k] = h[k];
    __syncthreads();

    if (!cifg) lstm_gate(p, sx, sh, p.w_i2i, p.w_r2i, p.w_c2i, c_in, p.b_i, ln, gi);
    lstm_gate(p, sx, sh, p.w_i2f, p.w_r2f, p.w_c2f, c_in, p.b_f, ln, gf);
    lstm_gate(p, sx, sh, p.w_i2c, p.w_r2c, nullptr, nullptr, p.b_c, ln, gc);
    if (ln) {
        if (!cifg) lstm_layer_norm(p, gi, p.ln_i, p.b_i, stats);
        lstm_layer_norm(p, gf, p.ln_f, p.b_f, stats);
        lstm_layer_norm(p, gc, p.ln_c, p.b_c, stats);
    }
    // every thread continues with the units it computed itself (layer norm, when enabled, has synchronised)
    for (int u = threadIdx.x; u < U; u += LSTM_THREADS) {
        const float f = lstm_act(gf[u], 6);
        float c = __fmul_rn(f, c_in[u]);
        if (p.activation > 0) gc[u] = lstm_act(gc[u], p.activation);
        const float gate = cifg ? __fsub_rn(1.0f, f) : lstm_act(gi[u], 6);
        c = __fadd_rn(c, __fmul_rn(gc[u], gate));
        if (p.cell_clip > 0.0f) c = lstm_clip(c, p.cell_clip);
        cn[u] = c;
        c_out[u] = c;
    }
    // the output gate's peephole term reads the new cell state of the same unit
    lstm_gate(p, sx, sh, p.w_i2o, p.w_r2o, p.w_c2o, cn, p.b_o, ln, go);
    if (ln) lstm_layer_norm(p, go, p.ln_o, p.b_o, stats);
    for (int u = threadIdx.x; u < U; u += LSTM_THREADS) {
        const float og = lstm_act(go[u], 6);
        // without an activation function the reference's cell scratch still holds the cell gate (Lstm.cpp:216-222)
        const float cs = p.activation > 0 ? lstm_act(cn[u], p.activation) : gc[u];
        go[u] = __fmul_rn(og, cs);
    }
    __syncthreads();
    if (p.w_proj) {
        for (int o = threadIdx.x; o < O; o += LSTM_THREADS) {
            float acc = p.b_proj ? p.b_proj[o] : 0.0f;
            const float* wrow = p.w_proj + (long long)o * U;
            for (int k = 0; k < U; ++k) acc = __fadd_rn(acc, __fmul_rn(wrow[k], go[k]));
            if (p.projection_clip > 0.0f) acc = lstm_clip(acc, p.projection_clip);
            out[o] = acc;
            p.output_state_out[(long long)b * O + o] = acc;
        }
    } else {
        for (int o = threadIdx.x; o < O; o += LSTM_THREADS) {
            out[o] = go[o];
            p.output_state_out[(long long)b * O + o] = go[o];
        }
    }
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_lstm_step_f32(const b200k_lstm_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "lstm_step_f32: null params");
    B200K_REQUIRE(p->batch > 0 && p->input_size > 0 && p->num_units > 0 && p->output_size > 0, B200K_E_INVALID, "lstm_step_f32: bad shape");
    B200K_REQUIRE(p->input && p->output_state_in && p->cell_state_in && p->output_state_out && p->cell_state_out && p->output,
                  B200K_E_INVALID, "lstm_step_f32: null state / input / output pointer");
    B200K_REQUIRE(p->w_i2f && p->w_i2c && p->w_i2o && p->w_r2f && p->w_r2c && p->w_r2o && p->b_f && p->b_c && p->b_o,
                  B200K_E_INVALID, "lstm_step_f32: a mandatory weight or bias is missing");
    const bool cifg = p->w_i2i == nullptr;
    B200K_REQUIRE(cifg || (p->w_r2i && p->b_i), B200K_E_INVALID, "lstm_step_f32: the input gate needs its recurrent weights and bias");
    B200K_REQUIRE(!p->w_c2f == !p->w_c2o && (cifg || !p->w_c2f == !p->w_c2i), B200K_E_INVALID, "lstm_step_f32: incomplete peephole weights");
    B200K_REQUIRE(!p->ln_f == !p->ln_c && !p->ln_f == !p->ln_o && (cifg || !p->ln_f == !p->ln_i), B200K_E_INVALID,
                  "lstm_step_f32: incomplete layer-norm weights");
    B200K_REQUIRE(p->w_proj || p->output_size == p->num_units, B200K_E_INVALID, "lstm_step_f32: without projection the output size is the number of units");
    B200K_REQUIRE(p->activation == 0 || p->activation == 1 || p->activation == 3 || p->activation == 4 || p->activation == 6,
                  B200K_E_UNSUPPORTED, "lstm_step_f32: unsupported activation function %d", p->activation);
    // The state tensors may be updated in place (the steps of a sequence do): a row's previous output is staged in
    // shared memory before anything is written, and a cell value is read and written by the same thread.
    const size_t smem = ((size_t)p->input_size + p->output_size + 5 * (size_t)p->num_units) * sizeof(float);
    B200K_REQUIRE(smem <= 200 * 1024, B200K_E_TOOBIG, "lstm_step_f32: %zu bytes of shared memory per row exceed 200 KiB", smem);
    static thread_local int opted_device = -1;
    if (smem > 48 * 1024) {
        int dev = 0;
        B200K_CUDA(cudaGetDevice(&dev));
        if (opted_device != dev) {
            B200K_CUDA(cudaFuncSetAttribute(lstm_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            opted_device = dev;
        }
    }
    launch_pdl(lstm_step_kernel, dim3((unsigned)p->batch), dim3(LSTM_THREADS), smem, (cudaStream_t)stream, *p);
    return check_launch("lstm_step_kernel");
}
