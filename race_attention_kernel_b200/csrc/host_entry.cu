// Host-buffer entry point: streams a causal forward whose tensors live in host memory through
// device staging buffers.  The sequence is cut into segments; segment i+1 is copied in while
// segment i computes and segment i-1 is copied out (three streams, two buffer sets), and the
// running state (A, B) stays on the device between segments -- the carried form of
// src/race_chunked.py:41-63 with the chunk loop turned into a copy/compute pipeline.
// The staging buffers, streams and events of a device are kept between calls (allocating and freeing
// about half a gigabyte of device memory per call costs more than the copies of a short sequence);
// race_b200_host_release() frees them.  Calls on the same device are serialised by a mutex.
#include <algorithm>
#include <mutex>

#include "launch.h"

using namespace race;

namespace {

struct HostPipe {
    cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr;
    cudaEvent_t in_done[2] = {nullptr, nullptr}, run_done[2] = {nullptr, nullptr},
                out_done[2] = {nullptr, nullptr};
    void* pq[2] = {nullptr, nullptr};
    void* pk[2] = {nullptr, nullptr};
    void* v[2] = {nullptr, nullptr};
    void* out[2] = {nullptr, nullptr};
    float* state[2] = {nullptr, nullptr};
    void* ws = nullptr;
    int* status = nullptr;   // device word the kernels raise when a bounded wait runs out
    size_t cap_probs = 0, cap_v = 0, cap_state = 0, cap_ws = 0;   // bytes each buffer holds
    std::mutex mu;

    void release_buffers() {
        for (int i = 0; i < 2; ++i) {
            cudaFree(pq[i]); cudaFree(pk[i]); cudaFree(v[i]); cudaFree(out[i]); cudaFree(state[i]);
            pq[i] = pk[i] = v[i] = out[i] = nullptr;
            state[i] = nullptr;
        }
        cudaFree(ws);
        ws = nullptr;
        cap_probs = cap_v = cap_state = cap_ws = 0;
    }
    void release_all() {
        release_buffers();
        for (int i = 0; i < 2; ++i) {
            if (in_done[i]) cudaEventDestroy(in_done[i]);
            if (run_done[i]) cudaEventDestroy(run_done[i]);
            if (out_done[i]) cudaEventDestroy(out_done[i]);
            in_done[i] = run_done[i] = out_done[i] = nullptr;
        }
        cudaFree(status);
        status = nullptr;
        if (s_in) cudaStreamDestroy(s_in);
        if (s_run) cudaStreamDestroy(s_run);
        if (s_out) cudaStreamDestroy(s_out);
        s_in = s_run = s_out = nullptr;
    }
};

#define RACE_TRY(expr)                                   \
    do {                                                 \
        cudaError_t e_ = (expr);                         \
        if (e_ != cudaSuccess) return (int)e_;           \
    } while (0)

constexpr int kMaxDevices = 64;
HostPipe g_pipes[kMaxDevices];   // never destroyed at exit: the context may be gone by then

// streams, events and the status word once; buffers whenever a call needs larger ones
int prepare(HostPipe& p, size_t probs_bytes, size_t v_bytes, size_t state_bytes, size_t ws_bytes) {
    if (!p.s_in) {
        RACE_TRY(cudaStreamCreateWithFlags(&p.s_in, cudaStreamNonBlocking));
        RACE_TRY(cudaStreamCreateWithFlags(&p.s_run, cudaStreamNonBlocking));
        RACE_TRY(cudaStreamCreateWithFlags(&p.s_out, cudaStreamNonBlocking));
        for (int i = 0; i < 2; ++i) {
            RACE_TRY(cudaEventCreateWithFlags(&p.in_done[i], cudaEventDisableTiming));
            RACE_TRY(cudaEventCreateWithFlags(&p.run_done[i], cudaEventDisableTiming));
            RACE_TRY(cudaEventCreateWithFlags(&p.out_done[i], cudaEventDisableTiming));
        }
        RACE_TRY(cudaMalloc((void**)&p.status, sizeof(int)));
    }
    if (probs_bytes > p.cap_probs || v_bytes > p.cap_v || state_bytes > p.cap_state || ws_bytes > p.cap_ws) {
        p.release_buffers();
        for (int i = 0; i < 2; ++i) {
            RACE_TRY(cudaMalloc(&p.pq[i], probs_bytes));
            RACE_TRY(cudaMalloc(&p.pk[i], probs_bytes));
            RACE_TRY(cudaMalloc(&p.v[i], v_bytes));
            RACE_TRY(cudaMalloc(&p.out[i], v_bytes));
            RACE_TRY(cudaMalloc((void**)&p.state[i], state_bytes));
        }
        RACE_TRY(cudaMalloc(&p.ws, ws_bytes));
        p.cap_probs = probs_bytes; p.cap_v = v_bytes; p.cap_state = state_bytes; p.cap_ws = ws_bytes;
    }
    return RACE_OK;
}

}  // namespace

extern "C" int race_b200_causal_fwd_host(const void* probs_q, const void* probs_k, const void* v,
                                         void* out, const float* carry_in, float* state_out,
                                         const RaceShape* shape, int64_t segment_tokens, int variant,
                                         int device) {
    if (!shape) return RACE_ERR_NULL;
    if (shape->n_streams <= 0 || shape->seq_len < 0) return shape->n_streams == 0 ? RACE_OK : RACE_ERR_SHAPE;
    if (shape->heads > 1) return RACE_ERR_SHAPE;   // segments are cut from contiguous [N, T, .] host tensors
    if (device < 0 || device >= kMaxDevices) return RACE_ERR_SHAPE;
    RACE_TRY(cudaSetDevice(device));
    RaceShape seg_shape = *shape;
    const int64_t N = shape->n_streams, T = shape->seq_len;
    const int64_t S = (int64_t)shape->n_tables * shape->n_buckets, D = shape->head_dim;
    const size_t eb = shape->dtype == RACE_DTYPE_BF16 ? 2 : 4;
    const size_t sf_bytes = (size_t)N * S * (D + 1) * sizeof(float);
    if (T > 0 && (!probs_q || !probs_k || !v || !out)) return RACE_ERR_NULL;

    // default segment: about 256 MB of tokens in flight per buffer set
    int64_t seg = segment_tokens;
    if (seg <= 0) {
        const int64_t per_token = N * (2 * S + 2 * D) * (int64_t)eb;
        seg = std::max<int64_t>(4096, ((int64_t)256 << 20) / per_token);
        seg = (seg + 2047) / 2048 * 2048;
    }
    seg = std::min<int64_t>(seg, std::max<int64_t>(T, 1));
    seg_shape.seq_len = seg;
    if (!race_b200_is_supported(&seg_shape, variant)) return RACE_ERR_SHAPE;
    // one tile length for every segment: a shorter last segment launched with the automatic choice
    // could pick a shorter tile and need more tile slices than the workspace holds
    int tile = 0;
    int rc0 = race_b200_select_tile_tokens(&seg_shape, variant, &tile);
    if (rc0 != RACE_OK) return rc0;
    size_t ws_bytes = race_b200_causal_workspace_bytes(&seg_shape, tile, variant);

    HostPipe& p = g_pipes[device];
    std::lock_guard<std::mutex> lock(p.mu);
    {
        const int rc = prepare(p, (size_t)N * seg * S * eb, (size_t)N * seg * D * eb, sf_bytes,
                               std::max<size_t>(ws_bytes, 256));
        if (rc != RACE_OK) { cudaGetLastError(); p.release_buffers(); return rc; }
    }

    // the pipeline proper; on any failure the copies already queued are allowed to finish before the
    // caller gets its buffers back
    auto run = [&]() -> int {
        // state[0] holds the carry into segment 0
        if (carry_in) RACE_TRY(cudaMemcpyAsync(p.state[0], carry_in, sf_bytes, cudaMemcpyHostToDevice, p.s_run));
        else RACE_TRY(cudaMemsetAsync(p.state[0], 0, sf_bytes, p.s_run));
        RACE_TRY(cudaMemsetAsync(p.status, 0, sizeof(int), p.s_run));

        const int64_t nseg = (T + seg - 1) / seg;
        for (int64_t i = 0; i < nseg; ++i) {
            const int b = (int)(i & 1);
            const int64_t t0 = i * seg, len = std::min<int64_t>(seg, T - t0);
            // copy in: [N rows] x [len*S elements] out of a host pitch of T*S elements
            if (i >= 2) RACE_TRY(cudaStreamWaitEvent(p.s_in, p.run_done[b], 0));
            RACE_TRY(cudaMemcpy2DAsync(p.pq[b], (size_t)len * S * eb, (const char*)probs_q + (size_t)t0 * S * eb,
                                       (size_t)T * S * eb, (size_t)len * S * eb, (size_t)N,
                                       cudaMemcpyHostToDevice, p.s_in));
            RACE_TRY(cudaMemcpy2DAsync(p.pk[b], (size_t)len * S * eb, (const char*)probs_k + (size_t)t0 * S * eb,
                                       (size_t)T * S * eb, (size_t)len * S * eb, (size_t)N,
                                       cudaMemcpyHostToDevice, p.s_in));
            RACE_TRY(cudaMemcpy2DAsync(p.v[b], (size_t)len * D * eb, (const char*)v + (size_t)t0 * D * eb,
                                       (size_t)T * D * eb, (size_t)len * D * eb, (size_t)N,
                                       cudaMemcpyHostToDevice, p.s_in));
            RACE_TRY(cudaEventRecord(p.in_done[b], p.s_in));

            // compute: carry state[i&1] -> state[(i+1)&1]
            RACE_TRY(cudaStreamWaitEvent(p.s_run, p.in_done[b], 0));
            if (i >= 2) RACE_TRY(cudaStreamWaitEvent(p.s_run, p.out_done[b], 0));
            seg_shape.seq_len = len;
            int rc = race_b200_causal_fwd(p.pq[b], p.pk[b], p.v[b], p.out[b], p.state[b], p.state[b ^ 1],
                                          p.ws, ws_bytes, &seg_shape, tile, variant, (void*)p.s_run, p.status);
            if (rc != RACE_OK) return rc;
            RACE_TRY(cudaEventRecord(p.run_done[b], p.s_run));

            // copy out
            RACE_TRY(cudaStreamWaitEvent(p.s_out, p.run_done[b], 0));
            RACE_TRY(cudaMemcpy2DAsync((char*)out + (size_t)t0 * D * eb, (size_t)T * D * eb, p.out[b],
                                       (size_t)len * D * eb, (size_t)len * D * eb, (size_t)N,
                                       cudaMemcpyDeviceToHost, p.s_out));
            RACE_TRY(cudaEventRecord(p.out_done[b], p.s_out));
        }
        if (state_out)
            RACE_TRY(cudaMemcpyAsync(state_out, p.state[nseg & 1], sf_bytes, cudaMemcpyDeviceToHost, p.s_run));
        int waited = 0;
        RACE_TRY(cudaMemcpyAsync(&waited, p.status, sizeof(int), cudaMemcpyDeviceToHost, p.s_run));
        RACE_TRY(cudaStreamSynchronize(p.s_in));
        RACE_TRY(cudaStreamSynchronize(p.s_run));
        RACE_TRY(cudaStreamSynchronize(p.s_out));
        return waited ? RACE_ERR_DEVICE_WAIT : RACE_OK;
    };
    const int rc = run();
    if (rc != RACE_OK) cudaDeviceSynchronize();
    return rc;
}

extern "C" int race_b200_host_release(int device) {
    if (device < 0 || device >= kMaxDevices) return RACE_ERR_SHAPE;
    HostPipe& p = g_pipes[device];
    std::lock_guard<std::mutex> lock(p.mu);
    if (!p.s_in && !p.ws) return RACE_OK;
    RACE_TRY(cudaSetDevice(device));
    p.release_all();
    return RACE_OK;
}
