// Decode layer-steps for a caller whose activations live in HOST memory: the three-stream pipeline
// (upload | kernels | download) behind the C ABI.
//
// The reference's engine keeps one decode thread that issues every launch in program order and synchronises
// once per layer (crates/engine/src/glm/forward.rs:276, crates/engine/src/glm/attn.rs:80-83); its stream and
// event wrappers (crates/backend/src/gpustream.rs:16-32) exist so that copies can overlap compute. This object is
// that idea for the one path of this library: a step's inputs travel as ONE packed pinned buffer (one copy per
// direction and step), `depth` device-side slots let the upload of step i + 1 and the download of step i - 1
// overlap the kernels of step i, and events order the slots; within a stream everything stays in program order,
// so results equal the serial order.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <new>
#include <vector>

#include "../../../include/rivoli_kernels.h"

#define RIVOLI_API extern "C" __attribute__((visibility("default")))

namespace {

size_t up256(size_t x) { return (x + 255) / 256 * 256; }

struct PackedLayout {
    size_t latent, index_key, index_q, index_w, q, total, out;
    PackedLayout(const DsaGeom& g, int B) {
        const size_t W = (size_t)g.kv_lora + g.rope_dim;
        size_t o = 0;
        latent = o;    o += up256((size_t)B * W * 2);
        index_key = o; o += up256((size_t)B * g.index_dim * 2);
        index_q = o;   o += up256((size_t)B * g.index_heads * g.index_dim * 2);
        index_w = o;   o += up256((size_t)B * g.index_heads * 4);
        q = o;         o += up256((size_t)B * g.n_heads * W * 2);
        total = o;
        out = (size_t)B * g.n_heads * g.kv_lora * 2;
    }
};

struct StepPipe {
    DsaGeom g;
    int B, depth;
    PackedLayout lay;
    std::vector<uint8_t*> in_slot, out_slot;
    cudaStream_t s_up = nullptr, s_run = nullptr, s_down = nullptr;
    std::vector<cudaEvent_t> ev_up0, ev_up, ev_run, ev_down;   // per slot: upload begin / end, kernels end, download end
    long long n = 0;
    StepPipe(const DsaGeom& g_, int B_, int depth_) : g(g_), B(B_), depth(depth_), lay(g_, B_) {}
};

int cu(cudaError_t e) { return e == cudaSuccess ? 0 : -(int)e; }

}  // namespace

RIVOLI_API size_t rivoli_step_pipe_input_bytes(const DsaGeom* g, int B) {
    return (g && B > 0) ? PackedLayout(*g, B).total : 0;
}
RIVOLI_API size_t rivoli_step_pipe_output_bytes(const DsaGeom* g, int B) {
    return (g && B > 0) ? PackedLayout(*g, B).out : 0;
}
RIVOLI_API int rivoli_step_pipe_input_offsets(const DsaGeom* g, int B, size_t off[5]) {
    if (!g || B <= 0 || !off) return 1001;
    const PackedLayout l(*g, B);
    off[0] = l.latent; off[1] = l.index_key; off[2] = l.index_q; off[3] = l.index_w; off[4] = l.q;
    return 0;
}

static void rivoli_step_pipe_destroy_impl(void* h) {
    StepPipe* p = static_cast<StepPipe*>(h);
    if (!p) return;
    if (p->s_up) cudaStreamSynchronize(p->s_up);
    if (p->s_run) cudaStreamSynchronize(p->s_run);
    if (p->s_down) cudaStreamSynchronize(p->s_down);
    for (auto x : p->in_slot) if (x) cudaFree(x);
    for (auto x : p->out_slot) if (x) cudaFree(x);
    for (auto* v : {&p->ev_up0, &p->ev_up, &p->ev_run, &p->ev_down})
        for (auto e : *v) if (e) cudaEventDestroy(e);
    if (p->s_up) cudaStreamDestroy(p->s_up);
    if (p->s_run) cudaStreamDestroy(p->s_run);
    if (p->s_down) cudaStreamDestroy(p->s_down);
    delete p;
}

// Allocates the device-side slots, three non-blocking streams and the events ONCE; a step allocates nothing.
RIVOLI_API void* rivoli_step_pipe_create(const DsaGeom* g, int B, int depth) {
    if (!g || B <= 0 || depth < 1 || depth > 8) return nullptr;
    StepPipe* p = new (std::nothrow) StepPipe(*g, B, depth);
    if (!p) return nullptr;
    bool ok = cudaStreamCreateWithFlags(&p->s_up, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&p->s_run, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&p->s_down, cudaStreamNonBlocking) == cudaSuccess;
    for (int i = 0; i < depth && ok; ++i) {
        uint8_t *a = nullptr, *b = nullptr;
        ok = cudaMalloc(&a, p->lay.total) == cudaSuccess && cudaMalloc(&b, p->lay.out) == cudaSuccess;
        p->in_slot.push_back(a); p->out_slot.push_back(b);
        cudaEvent_t e[4] = {};
        for (int k = 0; k < 4 && ok; ++k) ok = cudaEventCreate(&e[k]) == cudaSuccess;
        p->ev_up0.push_back(e[0]); p->ev_up.push_back(e[1]); p->ev_run.push_back(e[2]); p->ev_down.push_back(e[3]);
    }
    if (!ok) {
        rivoli_step_pipe_destroy_impl(p);
        return nullptr;
    }
    return p;
}

RIVOLI_API void rivoli_step_pipe_destroy(void* h) { rivoli_step_pipe_destroy_impl(h); }

// Enqueue one layer-step; never blocks the host. Returns a ticket (>= 0) for rivoli_step_pipe_wait, or a negative
// -(cudaError_t) / -(guard code) on failure.
RIVOLI_API long long rivoli_dsa_step_host(void* h, const DsaStepState* st, const void* host_in, void* host_out,
                                          const int32_t* row_pos, const int32_t* seq_len) {
    StepPipe* p = static_cast<StepPipe*>(h);
    if (!p || !st || !host_in || !host_out || !row_pos || !seq_len) return -1001;
    const int s = (int)(p->n % p->depth);
    const bool first = p->n < p->depth;
    int e = 0;
    if (!first) e = cu(cudaStreamWaitEvent(p->s_up, p->ev_run[s], 0));       // the step that last read this input slot is done
    if (!e) e = cu(cudaEventRecord(p->ev_up0[s], p->s_up));
    if (!e) e = cu(cudaMemcpyAsync(p->in_slot[s], host_in, p->lay.total, cudaMemcpyHostToDevice, p->s_up));
    if (!e) e = cu(cudaEventRecord(p->ev_up[s], p->s_up));
    if (!e) e = cu(cudaStreamWaitEvent(p->s_run, p->ev_up[s], 0));
    if (!e && !first) e = cu(cudaStreamWaitEvent(p->s_run, p->ev_down[s], 0));  // this output slot has been downloaded
    if (e) return e;
    const uint8_t* in = p->in_slot[s];
    const int r = rivoli_dsa_decode_step_paged(
        &p->g, reinterpret_cast<const uint16_t*>(in + p->lay.latent), reinterpret_cast<const uint16_t*>(in + p->lay.index_key),
        row_pos, st->block_table, st->latent_pool, st->latent_scale, st->index_pool, st->index_scale, st->status,
        reinterpret_cast<const uint16_t*>(in + p->lay.index_q), reinterpret_cast<const float*>(in + p->lay.index_w), seq_len,
        p->B, st->score_stride, st->rows, st->n_sel, st->select_scratch, reinterpret_cast<const uint16_t*>(in + p->lay.q),
        reinterpret_cast<uint16_t*>(p->out_slot[s]), st->out_m, st->out_lse, st->attend_scratch, st->min_rows_hint, p->s_run);
    if (r) return r > 0 ? -(long long)r : r;
    e = cu(cudaEventRecord(p->ev_run[s], p->s_run));
    if (!e) e = cu(cudaStreamWaitEvent(p->s_down, p->ev_run[s], 0));
    if (!e) e = cu(cudaMemcpyAsync(host_out, p->out_slot[s], p->lay.out, cudaMemcpyDeviceToHost, p->s_down));
    if (!e) e = cu(cudaEventRecord(p->ev_down[s], p->s_down));
    if (e) return e;
    return p->n++;
}

// Blocks until the output of step `ticket` is in its host buffer.
RIVOLI_API int rivoli_step_pipe_wait(void* h, long long ticket) {
    StepPipe* p = static_cast<StepPipe*>(h);
    if (!p || ticket < 0 || ticket >= p->n) return 1001;
    // the slot's event belongs to this step or, if the slot was reused, to a later download on the same
    // in-order stream, whose completion implies this one's
    return cu(cudaEventSynchronize(p->ev_down[ticket % p->depth]));
}
RIVOLI_API int rivoli_step_pipe_drain(void* h) {
    StepPipe* p = static_cast<StepPipe*>(h);
    if (!p) return 1001;
    return cu(cudaStreamSynchronize(p->s_down));
}
// Milliseconds of the three legs of the LAST completed use of every slot, averaged over the slots:
// ms[0] upload, ms[1] upload end -> kernels end, ms[2] kernels end -> download end. Synchronises the pipeline.
RIVOLI_API int rivoli_step_pipe_leg_ms(void* h, float ms[3]) {
    StepPipe* p = static_cast<StepPipe*>(h);
    if (!p || !ms || p->n < p->depth) return 1001;
    if (int e = rivoli_step_pipe_drain(h)) return e;
    ms[0] = ms[1] = ms[2] = 0.0f;
    for (int s = 0; s < p->depth; ++s) {
        float a = 0, b = 0, c = 0;
        if (int e = cu(cudaEventElapsedTime(&a, p->ev_up0[s], p->ev_up[s]))) return e;
        if (int e = cu(cudaEventElapsedTime(&b, p->ev_up[s], p->ev_run[s]))) return e;
        if (int e = cu(cudaEventElapsedTime(&c, p->ev_run[s], p->ev_down[s]))) return e;
        ms[0] += a / p->depth; ms[1] += b / p->depth; ms[2] += c / p->depth;
    }
    return 0;
}
// The streams, for a caller that wants to bracket a run with its own events: which = 0 upload, 1 kernels, 2 download.
RIVOLI_API void* rivoli_step_pipe_stream(void* h, int which) {
    StepPipe* p = static_cast<StepPipe*>(h);
    if (!p) return nullptr;
    return which == 0 ? p->s_up : (which == 1 ? p->s_run : p->s_down);
}
