/*
 * tp.cu - tensor-parallel plumbing of the fused FFN: the per-rank exchange buffer the down
 * projection's epilogue writes into on every peer, how ranks learn each other's buffers (CUDA IPC
 * between processes, peer access inside one process), and the operator entry that runs one rank's
 * FFN with the in-kernel reduce.  Replaces the reference's peer_probe_all / allreduce_sum pair
 * (csrc/collective.cu:108-144, 168-219) for this path: no staging copies, no host-issued adds.
 *
 * One exchange buffer per rank, one allocation:
 *     [ call counter u32, pad | slots: 2 x tp x max_tokens*hidden x {f32 value, u32 call number + 1} ]
 * Every element travels as one 8-byte store whose upper half names the call it belongs to; the
 * receiver polls the element itself.  The kernel takes the call number from a device-resident
 * counter, so replaying a captured graph stays correct.  Slots are double buffered by call parity:
 * a rank can be at most one call ahead of a peer, because completing a call needs every peer's
 * elements of that call.
 */
#include <string.h>

#include <new>

#include "common.cuh"
#include "kernels.h"

namespace ffn {


struct TpComm {
    int tp = 0, rank = 0, hidden = 0, max_tokens = 0, device = 0;
    size_t bytes = 0;
    uint8_t *local = nullptr;             /* this rank's exchange buffer */
    uint8_t *peer[kTpMaxRanks] = {};      /* every rank's buffer as seen from this device */
    bool opened[kTpMaxRanks] = {};        /* peer[r] came from cudaIpcOpenMemHandle */
    unsigned long long **d_slots = nullptr; /* device array handed to the kernel */
    bool connected = false;
};

/* Puts the calling thread's current device back when a function that switches devices returns. */
struct DeviceRestore {
    int dev = -1;
    DeviceRestore() { if (cudaGetDevice(&dev) != cudaSuccess) { dev = -1; (void)cudaGetLastError(); } }
    ~DeviceRestore() { if (dev >= 0) (void)cudaSetDevice(dev); }
};

static int tp_publish_tables(TpComm *c) {
    unsigned long long *slots[kTpMaxRanks];
    for (int r = 0; r < c->tp; ++r) slots[r] = (unsigned long long *)(c->peer[r] + kTpHeaderBytes);
    if (!c->d_slots && cudaMalloc(&c->d_slots, sizeof(slots)) != cudaSuccess)
        return fail(FFN_ERR_ALLOC, "ffn_tp: cannot allocate the peer table");
    FFN_CUDA_TRY(cudaMemcpy(c->d_slots, slots, sizeof(slots), cudaMemcpyHostToDevice), "ffn_tp: peer table");
    c->connected = true;
    return FFN_OK;
}

/* Stand-alone all-reduce over the communicator's exchange slots: every thread pushes its elements
 * (as FP32) into slot `rank` of every rank's buffer, then waits (bounded) for the tp words of each
 * of its elements in its own buffer, adds them in rank order and stores the rounded sum in place. */
template <typename T> struct ElemIo;
template <> struct ElemIo<float> {
    static __device__ __forceinline__ float load(const float *p) { return *p; }
    static __device__ __forceinline__ void store(float *p, float v) { *p = v; }
};
template <> struct ElemIo<uint16_t> { /* bf16 bits */
    static __device__ __forceinline__ float load(const uint16_t *p) { return bf16_bits_to_f32(*p); }
    static __device__ __forceinline__ void store(uint16_t *p, float v) { *p = f32_to_bf16_bits(v); }
};

template <typename T>
__global__ void tp_allreduce_kernel(T *buf, size_t elements, unsigned long long *const *peer_slots, int slot_stride,
                                    int tp, int rank, const unsigned *seq_word, unsigned *status) {
    const unsigned seq = *seq_word; /* advanced by the launch that follows this one on the stream */
    const unsigned tag = tp_tag(seq);
    const size_t par = (size_t)(seq & 1u) * tp * slot_stride;
    const size_t stride = (size_t)gridDim.x * blockDim.x, first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (size_t i = first; i < elements; i += stride) {
        const float v = ElemIo<T>::load(buf + i);
        for (int r = 0; r < tp; ++r) tp_store_tagged(peer_slots[r] + par + (size_t)rank * slot_stride + i, v, tag);
    }
    const unsigned long long *mine = peer_slots[rank] + par;
    for (size_t i = first; i < elements; i += stride) {
        float sum = 0.0f;
        bool all_in = true;
        for (int r = 0; r < tp && all_in; ++r) {
            const unsigned long long *p = mine + (size_t)r * slot_stride + i;
            float v = 0.0f;
            bool in = tp_load_tagged(p, tag, &v);
            for (uint32_t k = 0; !in && k < kTpPollLimit; ++k) {
                __nanosleep(40);
                in = tp_load_tagged(p, tag, &v);
            }
            all_in = in;
            sum += v;
        }
        if (!all_in) { atomicCAS(status, 0u, 6u | ((unsigned)blockIdx.x << 8)); return; } /* 6 = a peer rank's data */
        ElemIo<T>::store(buf + i, sum);
    }
}
__global__ void tp_seq_advance_kernel(unsigned *seq_word) { *seq_word += 1u; }

static int tp_allreduce_launch(TpComm *c, cudaStream_t stream, void *buffer, size_t elements, int dtype) {
    if (!c->connected) return fail(FFN_ERR_STATE, "ffn_tp_allreduce_sum: the communicator is not connected");
    if (dtype != 0 && dtype != 2) return fail(FFN_ERR_CONFIG, "ffn_tp_allreduce_sum: unknown element type %d (0 = f32, 2 = bf16)", dtype);
    if (elements == 0) return FFN_OK;
    if (!buffer) return fail(FFN_ERR_CONFIG, "ffn_tp_allreduce_sum: null buffer");
    const size_t cap = (size_t)c->max_tokens * c->hidden;
    if (elements > cap) return fail(FFN_ERR_CONFIG, "ffn_tp_allreduce_sum: %zu elements exceed the exchange slots (%zu)", elements, cap);
    if (c->tp == 1) return FFN_OK;
    unsigned *status = nullptr;
    int st = fused_status_word(&status);
    if (st) return st;
    int sms = 0;
    FFN_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device), "SM count");
    const int threads = 256;
    const int blocks = (int)min((size_t)sms * 4, (elements + threads - 1) / threads);
    unsigned *seq = (unsigned *)(c->local + kTpSeqOffset);
    if (dtype == 0)
        tp_allreduce_kernel<float><<<blocks, threads, 0, stream>>>((float *)buffer, elements, c->d_slots, c->max_tokens * c->hidden, c->tp, c->rank, seq, status);
    else
        tp_allreduce_kernel<uint16_t><<<blocks, threads, 0, stream>>>((uint16_t *)buffer, elements, c->d_slots, c->max_tokens * c->hidden, c->tp, c->rank, seq, status);
    FFN_CUDA_TRY(cudaGetLastError(), "ffn_tp_allreduce_sum launch");
    tp_seq_advance_kernel<<<1, 1, 0, stream>>>(seq);
    FFN_CUDA_TRY(cudaGetLastError(), "ffn_tp_allreduce_sum launch");
    return FFN_OK;
}

}  // namespace ffn

using namespace ffn;

extern "C" {

int ffn_tp_create(FfnTpComm **out, int tp, int rank, int hidden, int max_tokens) {
    clear_error();
    if (!out) return fail(FFN_ERR_CONFIG, "ffn_tp_create: null argument");
    if (tp < 1 || tp > kTpMaxRanks || rank < 0 || rank >= tp)
        return fail(FFN_ERR_CONFIG, "ffn_tp_create: rank %d is outside [0, %d) or more than %d ranks", rank, tp, kTpMaxRanks);
    if (hidden <= 0 || hidden % FFN_INT4_GROUP || max_tokens < 1)
        return fail(FFN_ERR_CONFIG, "ffn_tp_create: invalid hidden size or token bound");
    TpComm *c = new (std::nothrow) TpComm();
    if (!c) return fail(FFN_ERR_ALLOC, "ffn_tp_create: out of host memory");
    c->tp = tp; c->rank = rank; c->hidden = hidden; c->max_tokens = max_tokens;
    if (cudaGetDevice(&c->device) != cudaSuccess) { delete c; return fail(FFN_ERR_CUDA, "ffn_tp_create: no CUDA device"); }
    c->bytes = kTpHeaderBytes + (size_t)2 * tp * max_tokens * hidden * sizeof(unsigned long long);
    if (cudaMalloc(&c->local, c->bytes) != cudaSuccess) {
        (void)cudaGetLastError();
        delete c;
        return fail(FFN_ERR_ALLOC, "ffn_tp_create: cannot allocate the %zu-byte exchange buffer", c->bytes);
    }
    if (cudaMemset(c->local, 0, c->bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
        cudaFree(c->local);
        delete c;
        return fail(FFN_ERR_CUDA, "ffn_tp_create: cannot clear the exchange buffer");
    }
    c->peer[rank] = c->local;
    *out = (FfnTpComm *)c;
    if (tp == 1) return tp_publish_tables(c);
    return FFN_OK;
}

int ffn_tp_export(FfnTpComm *comm, void *handle_out) {
    clear_error();
    TpComm *c = (TpComm *)comm;
    if (!c || !handle_out) return fail(FFN_ERR_CONFIG, "ffn_tp_export: null argument");
    cudaIpcMemHandle_t h;
    FFN_CUDA_TRY(cudaIpcGetMemHandle(&h, c->local), "ffn_tp_export: cudaIpcGetMemHandle");
    static_assert(sizeof(h) == FFN_TP_HANDLE_BYTES, "IPC handle size");
    memcpy(handle_out, &h, sizeof(h));
    return FFN_OK;
}

int ffn_tp_connect(FfnTpComm *comm, const void *all_handles) {
    clear_error();
    TpComm *c = (TpComm *)comm;
    if (!c || !all_handles) return fail(FFN_ERR_CONFIG, "ffn_tp_connect: null argument");
    if (c->connected) return fail(FFN_ERR_STATE, "ffn_tp_connect: already connected");
    DeviceRestore restore_device;
    FFN_CUDA_TRY(cudaSetDevice(c->device), "ffn_tp_connect: select device");
    for (int r = 0; r < c->tp; ++r) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t *)all_handles + (size_t)r * FFN_TP_HANDLE_BYTES, sizeof(h));
        void *p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            return fail(FFN_ERR_CUDA, "ffn_tp_connect: rank %d cannot map rank %d's exchange buffer: %s", c->rank, r,
                        cudaGetErrorString(e));
        }
        c->peer[r] = (uint8_t *)p;
        c->opened[r] = true;
    }
    return tp_publish_tables(c);
}

int ffn_tp_connect_local(FfnTpComm *const *comms, int count) {
    clear_error();
    if (!comms || count < 1 || count > kTpMaxRanks) return fail(FFN_ERR_CONFIG, "ffn_tp_connect_local: bad arguments");
    for (int i = 0; i < count; ++i) {
        TpComm *c = (TpComm *)comms[i];
        if (!c || c->tp != count || c->rank != i) return fail(FFN_ERR_CONFIG, "ffn_tp_connect_local: element %d is not rank %d of %d", i, i, count);
    }
    DeviceRestore restore_device;
    for (int i = 0; i < count; ++i) {
        TpComm *c = (TpComm *)comms[i];
        FFN_CUDA_TRY(cudaSetDevice(c->device), "ffn_tp_connect_local: select device");
        for (int j = 0; j < count; ++j) {
            TpComm *o = (TpComm *)comms[j];
            c->peer[j] = o->local;
            if (i == j || o->device == c->device) continue;
            int can = 0;
            FFN_CUDA_TRY(cudaDeviceCanAccessPeer(&can, c->device, o->device), "ffn_tp_connect_local: peer query");
            if (!can) return fail(FFN_ERR_CONFIG, "ffn_tp_connect_local: device %d cannot reach device %d", c->device, o->device);
            const cudaError_t e = cudaDeviceEnablePeerAccess(o->device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
                return fail(FFN_ERR_CUDA, "ffn_tp_connect_local: peer access %d->%d: %s", c->device, o->device, cudaGetErrorString(e));
            (void)cudaGetLastError(); /* "already enabled" is sticky (csrc/collective.cu:127-131) */
        }
        const int st = tp_publish_tables(c);
        if (st) return st;
    }
    return FFN_OK;
}

int ffn_tp_destroy(FfnTpComm *comm) {
    clear_error();
    TpComm *c = (TpComm *)comm;
    if (!c) return FFN_OK;
    DeviceRestore restore_device;
    (void)cudaSetDevice(c->device);
    (void)cudaDeviceSynchronize();
    for (int r = 0; r < c->tp; ++r)
        if (c->opened[r]) (void)cudaIpcCloseMemHandle(c->peer[r]);
    if (c->d_slots) cudaFree(c->d_slots);
    if (c->local) cudaFree(c->local);
    delete c;
    (void)cudaGetLastError();
    return FFN_OK;
}

int ffn_forward_mlp_tp(FfnTpComm *comm, void *stream, const void *normed, void *ws, void *layer_out,
                       const FfnMlpWeights *w, int tokens, const FfnModelDims *dims, void *residual) {
    clear_error();
    TpComm *c = (TpComm *)comm;
    if (!c || !w || !dims || !normed || !ws || !layer_out) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_tp: null argument");
    if (!c->connected) return fail(FFN_ERR_STATE, "ffn_forward_mlp_tp: the communicator is not connected");
    if (dims->hidden_size != c->hidden) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_tp: hidden size %d, communicator built for %d", dims->hidden_size, c->hidden);
    if (tokens < 1 || tokens > c->max_tokens || tokens > 64) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_tp: %d tokens, communicator built for at most %d", tokens, c->max_tokens);
    if (!w->gate_up_i4 || !w->gate_up_i4_scales || !w->down_i4 || !w->down_i4_scales || w->i4_group != FFN_INT4_GROUP)
        return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_tp: the layer carries no INT4 operands");
    const int H = dims->hidden_size, I = dims->intermediate_size;
    if (I <= 0 || I % FFN_INT4_GROUP) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_tp: the rank's intermediate size %d splits K at a non-group boundary", I);
    FusedTp t;
    t.tp = c->tp; t.rank = c->rank;
    t.peer_slots = c->d_slots;
    t.slot_stride = c->max_tokens * c->hidden;
    t.seq = (unsigned *)(c->local + kTpSeqOffset);
    uint16_t *act = (uint16_t *)ws + (size_t)tokens * H + (size_t)2 * tokens * I;
    int st = fused_ffn_launch((cudaStream_t)stream, normed, act, layer_out, w, tokens, H, I, &t, residual, nullptr);
    if (st == FFN_NOT_ADMITTED && tokens <= 64) {
        unsigned *status = nullptr;
        if ((st = fused_status_word(&status))) return st;
        st = batched_ffn_launch((cudaStream_t)stream, normed, act, layer_out, w, tokens, H, I, &t, residual, status);
    }
    if (st == FFN_NOT_ADMITTED)
        return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_tp: the fused kernel does not take this shape (tokens=%d H=%d I=%d)", tokens, H, I);
    return st;
}


int ffn_tp_allreduce_sum(FfnTpComm *comm, void *stream, void *buffer, size_t elements, int dtype) {
    clear_error();
    TpComm *c = (TpComm *)comm;
    if (!c) return fail(FFN_ERR_CONFIG, "ffn_tp_allreduce_sum: null communicator");
    return tp_allreduce_launch(c, (cudaStream_t)stream, buffer, elements, dtype);
}

int ffn_allreduce_sum(FfnTpComm *const *comms, void *const *streams, int count, void *const *buffers, size_t elements,
                      int dtype) {
    clear_error();
    if (count < 0 || !comms || !buffers) return fail(FFN_ERR_CONFIG, "ffn_allreduce_sum: null argument or negative count");
    if (count <= 1 || elements == 0) return FFN_OK; /* as the reference: nothing to do */
    for (int i = 0; i < count; ++i) {
        TpComm *c = (TpComm *)comms[i];
        if (!c || c->tp != count || c->rank != i) return fail(FFN_ERR_CONFIG, "ffn_allreduce_sum: element %d is not rank %d of %d", i, i, count);
    }
    DeviceRestore restore_device;
    int st = FFN_OK;
    for (int i = 0; i < count && !st; ++i) {
        TpComm *c = (TpComm *)comms[i];
        if (cudaSetDevice(c->device) != cudaSuccess) { st = fail(FFN_ERR_CUDA, "ffn_allreduce_sum: cannot select device %d", c->device); break; }
        st = tp_allreduce_launch(c, streams ? (cudaStream_t)streams[i] : nullptr, buffers[i], elements, dtype);
    }
    return st;
}

/* The input of a host-buffer call, fetched from mapped host memory by one small CTA: a few
 * microseconds of PCIe reads in flight together, where a copy-engine transfer costs its own start-up
 * and a hand-over between the copy engine and the compute queue. */
__global__ void stage_host_input_kernel(uint4 *__restrict__ dst, const uint4 *__restrict__ src_mapped, int chunks) {
    /* The FFN kernel that follows is launched with the dependent-launch attribute: let it start now
     * (barrier set-up, first weight copies); it waits for this grid before it reads the input. */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (int i = threadIdx.x; i < chunks; i += blockDim.x) dst[i] = src_mapped[i];
}

int ffn_forward_mlp_host(FfnTpComm *comm, void *stream, const void *normed_host, void *layer_out_host, void *staging,
                         void *ws, const FfnMlpWeights *w, int tokens, const FfnModelDims *dims) {
    clear_error();
    if (!dims || !w) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_host: null weights or dims");
    if (!normed_host || !layer_out_host || !staging || !ws) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_host: null buffer");
    const int limit = dims->max_chunk > 0 ? dims->max_chunk : 128;
    if (tokens < 1 || tokens > limit) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_host: Layer token count exceeds the model's max_chunk");
    if (dims->hidden_size <= 0) return fail(FFN_ERR_CONFIG, "ffn_forward_mlp_host: invalid hidden size");
    const size_t bytes = (size_t)tokens * dims->hidden_size * 2;
    cudaStream_t s = (cudaStream_t)stream;
    /* Pinned (or registered) host memory is mapped into the device's address space: the kernel can
     * write its results across PCIe itself, which costs less than a copy call.  Pageable memory goes
     * through `staging`. */
    auto mapped = [](const void *p) -> void * {
        cudaPointerAttributes attr;
        if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
        if (attr.type == cudaMemoryTypeUnregistered) return nullptr;
        return attr.devicePointer; /* device and managed memory: the pointer itself */
    };
    /* The input is read by every CTA, so it is copied to the device once; the output is written once,
     * by the CTAs that own its rows, and can go straight to mapped host memory. */
    uint16_t *x_dev = (uint16_t *)staging, *y_dev = (uint16_t *)mapped(layer_out_host);
    const bool stage_out = y_dev == nullptr;
    const void *x_mapped = mapped(normed_host);
    if (x_mapped && bytes <= (64u << 10) && !(((uintptr_t)x_mapped | (uintptr_t)x_dev) & 15)) {
        stage_host_input_kernel<<<1, 512, 0, s>>>((uint4 *)x_dev, (const uint4 *)x_mapped, (int)(bytes / 16));
        FFN_CUDA_TRY(cudaGetLastError(), "ffn_forward_mlp_host: input staging launch");
    } else {
        FFN_CUDA_TRY(cudaMemcpyAsync(x_dev, normed_host, bytes, cudaMemcpyDefault, s), "ffn_forward_mlp_host: input copy");
    }
    if (stage_out) y_dev = (uint16_t *)staging + (size_t)tokens * dims->hidden_size;
    TpComm *c = (TpComm *)comm;
    const int st = (c && c->tp > 1) ? ffn_forward_mlp_tp(comm, stream, x_dev, ws, y_dev, w, tokens, dims, nullptr)
                                    : ffn_forward_mlp_prepared(nullptr, stream, x_dev, ws, y_dev, w, tokens, dims);
    if (st) return st;
    if (stage_out) FFN_CUDA_TRY(cudaMemcpyAsync(layer_out_host, y_dev, bytes, cudaMemcpyDefault, s), "ffn_forward_mlp_host: output copy");
    FFN_CUDA_TRY(cudaStreamSynchronize(s), "ffn_forward_mlp_host: synchronize");
    return FFN_OK;
}

/* One layer of the decode stack: h <- bf16(h + FFN(RMSNorm(h))) */
static int decode_layer(TpComm *c, cudaStream_t stream, void *h, void *ws, void *layer_out, const FfnMlpWeights *w,
                        int tokens, const FfnModelDims *dims) {
    const int H = dims->hidden_size, I = dims->intermediate_size;
    if (!w->gate_up_i4 || !w->gate_up_i4_scales || !w->down_i4 || !w->down_i4_scales || w->i4_group != FFN_INT4_GROUP)
        return fail(FFN_ERR_CONFIG, "ffn_decode_layer: the layer carries no INT4 operands");
    if (!w->post_norm_w) return fail(FFN_ERR_CONFIG, "ffn_decode_layer: the layer has no post-norm weight");
    if (!(dims->rms_eps > 0.0f)) return fail(FFN_ERR_CONFIG, "ffn_decode_layer: invalid shape or epsilon");
    FusedTp t = {};
    const FusedTp *tp = nullptr;
    if (c && c->tp > 1) {
        t.tp = c->tp; t.rank = c->rank; t.peer_slots = c->d_slots;
        t.slot_stride = c->max_tokens * c->hidden; t.seq = (unsigned *)(c->local + kTpSeqOffset);
        tp = &t;
    }
    uint16_t *normed = (uint16_t *)ws;
    uint16_t *act = normed + (size_t)tokens * H + (size_t)2 * tokens * I;
    FusedNorm norm = {w->post_norm_w, dims->rms_eps, dims->norm_style == 0};
    /* 1-2 tokens: norm, FFN, cross-rank reduce and residual update in ONE launch */
    int st = fused_ffn_launch(stream, h, act, layer_out, w, tokens, H, I, tp, h, &norm);
    if (st != FFN_NOT_ADMITTED) return st;
    if (tokens > 64) return fail(FFN_ERR_CONFIG, "ffn_decode_layer: at most 64 tokens per call");
    st = gemma_rms_norm(normed, h, w->post_norm_w, H, tokens, dims->rms_eps, dims->norm_style == 0, stream);
    if (st) return st;
    unsigned *status = nullptr;
    if ((st = fused_status_word(&status))) return st;
    st = batched_ffn_launch(stream, normed, act, layer_out, w, tokens, H, I, tp, h, status);
    if (st == FFN_NOT_ADMITTED) return fail(FFN_ERR_CONFIG, "ffn_decode_layer: no kernel takes tokens=%d H=%d I=%d", tokens, H, I);
    return st;
}

int ffn_decode_stack(FfnTpComm *comm, void *stream, void *h, void *ws, void *layer_out, const FfnMlpWeights *layers,
                     int num_layers, int tokens, const FfnModelDims *dims) {
    clear_error();
    TpComm *c = (TpComm *)comm;
    if (!h || !ws || !layer_out || !layers || !dims) return fail(FFN_ERR_CONFIG, "ffn_decode_stack: null argument");
    if (num_layers < 0) return fail(FFN_ERR_CONFIG, "ffn_decode_stack: negative layer count");
    if (c && !c->connected) return fail(FFN_ERR_STATE, "ffn_decode_stack: the communicator is not connected");
    if (c && c->tp > 1 && (dims->hidden_size != c->hidden || tokens > c->max_tokens))
        return fail(FFN_ERR_CONFIG, "ffn_decode_stack: the communicator was built for hidden %d and at most %d tokens", c->hidden, c->max_tokens);
    const int limit = dims->max_chunk > 0 ? dims->max_chunk : 128;
    if (tokens < 1 || tokens > limit) return fail(FFN_ERR_CONFIG, "ffn_decode_stack: Layer token count exceeds the model's max_chunk");
    const int H = dims->hidden_size, I = dims->intermediate_size;
    if (H <= 0 || I <= 0 || H % FFN_INT4_GROUP || I % FFN_INT4_GROUP)
        return fail(FFN_ERR_CONFIG, "ffn_decode_stack: hidden=%d / intermediate=%d are not whole numbers of %d-wide groups", H, I, FFN_INT4_GROUP);
    if (tokens <= 4 && num_layers > 0) {
        /* every layer prepared with ffn_decode_layer_prepare: the whole stack in one persistent launch per 64 layers */
        bool whole = dims->rms_eps > 0.0f;
        for (int l = 0; l < num_layers && whole; ++l)
            whole = layers[l].gate_up_i4 && layers[l].gate_up_i4_scales && layers[l].down_i4 && layers[l].down_i4_scales &&
                    layers[l].i4_group == FFN_INT4_GROUP && layers[l].post_norm_w;
        if (whole) {
            FusedTp t = {};
            const FusedTp *tp = nullptr;
            if (c && c->tp > 1) {
                t.tp = c->tp; t.rank = c->rank; t.peer_slots = c->d_slots;
                t.slot_stride = c->max_tokens * c->hidden; t.seq = (unsigned *)(c->local + kTpSeqOffset);
                tp = &t;
            }
            unsigned *status = nullptr;
            int st = fused_status_word(&status);
            if (st) return st;
            uint16_t *act = (uint16_t *)ws + (size_t)tokens * H + (size_t)2 * tokens * I;
            st = kmajor_ffn_launch((cudaStream_t)stream, h, act, layer_out, layers, num_layers, tokens, H, I, tp, h, 1, dims->rms_eps,
                                   dims->norm_style == 0, status);
            if (st != FFN_NOT_ADMITTED) return st;
        }
    }
    for (int l = 0; l < num_layers; ++l) {
        const int st = decode_layer(c, (cudaStream_t)stream, h, ws, layer_out, layers + l, tokens, dims);
        if (st) return st;
    }
    return FFN_OK;
}

}  // extern "C"
