// Host-buffer entry points: the caller hands over HOST pointers, the library stages the data
// through device buffers it owns.  This is the call the end-to-end benchmark times: the batch is
// cut into chunks, each chunk travels host -> device, runs forward + backward and returns
// device -> host on its own stream, so that the copies of one chunk overlap the kernels of another
// (both copy engines and the SMs stay busy).  Inputs should be page-locked for the copies to be
// asynchronous; pageable memory works but serialises.
//
// A plan belongs to the device that was current when it was created; calls with another current
// device are refused.  Nothing here throws across the C boundary: the plan is a plain struct
// with fixed-size arrays, allocated with new(std::nothrow).
#include "internal.cuh"
#include <new>

using namespace cxxattn;

namespace {

constexpr int kMaxSlots = 4;
constexpr int kMaxBufs = 9;

// Device buffers, workspace and stream of one chunk in flight.
struct Slot {
    cudaStream_t st;
    char* buf[kMaxBufs];
    float* aux;  // softmax: row statistics; linear: den
    void* ws;
};

void free_slots(Slot* slots, int n) {
    for (int i = 0; i < n; i++) {
        for (char* b : slots[i].buf) cudaFree(b);
        cudaFree(slots[i].aux);
        cudaFree(slots[i].ws);
        if (slots[i].st) cudaStreamDestroy(slots[i].st);
    }
}

// nbuf buffers of buf_bytes, aux_bytes of floats and ws_bytes of workspace per slot.
bool alloc_slots(Slot* slots, int n, int nbuf, size_t buf_bytes, size_t aux_bytes, size_t ws_bytes) {
    for (int i = 0; i < n; i++) slots[i] = Slot{};
    for (int i = 0; i < n; i++) {
        Slot& s = slots[i];
        bool ok = cudaStreamCreateWithFlags(&s.st, cudaStreamNonBlocking) == cudaSuccess;
        for (int b = 0; b < nbuf && ok; b++) ok = cudaMalloc(&s.buf[b], buf_bytes) == cudaSuccess;
        ok = ok && cudaMalloc(&s.aux, aux_bytes) == cudaSuccess;
        ok = ok && (ws_bytes == 0 || cudaMalloc(&s.ws, ws_bytes) == cudaSuccess);
        if (!ok) return false;
    }
    return true;
}

// Waits for every slot; a CUDA failure or a device-side wait that gave up turns a good `rc` bad.
int drain(Slot* slots, int n, int rc) {
    for (int i = 0; i < n; i++)
        if (cudaStreamSynchronize(slots[i].st) != cudaSuccess && rc == CXXATTN_OK) rc = CXXATTN_ERR_CUDA;
    // the caller has no stream of its own to ask: report a timed-out device wait here (the tensor-core
    // kernels of any slot record it in the one status word of the device)
    const int st = sync_status(nullptr);
    return rc == CXXATTN_OK ? st : rc;
}

}  // namespace

struct cxxattn_host_plan {
    cxxattn_mha_desc desc;  // whole problem, reference layout
    int device;
    int chunk_b;            // batch items per chunk
    int nslots;
    size_t elem;            // bytes per element
    size_t chunk_elems;     // elements of one tensor of one full chunk
    size_t ws_bytes;
    Slot slots[kMaxSlots];  // buf: Q K V dO O dQ dK dV
};

struct cxxattn_lin_host_plan {
    cxxattn_lin_desc desc;  // whole problem
    int device;
    int chunk_b;            // units per chunk
    int nslots;
    size_t elem;
    size_t ws_bytes;
    Slot slots[kMaxSlots];  // buf: Q K V dO O dQ dK dV
};

extern "C" {

void cxxattn_host_plan_destroy(cxxattn_host_plan* plan) {
    if (plan == nullptr) return;
    free_slots(plan->slots, plan->nslots);
    delete plan;
}

int cxxattn_host_plan_create(cxxattn_host_plan** out, const cxxattn_mha_desc* desc, int batch_per_chunk) {
    if (out == nullptr || desc == nullptr || batch_per_chunk <= 0) return CXXATTN_ERR_INVALID;
    if (desc->B <= 0 || desc->S <= 0 || desc->H <= 0 || desc->Dh <= 0 || desc->reserved != 0) return CXXATTN_ERR_INVALID;
    if (desc->stride_b || desc->stride_s || desc->stride_h) return CXXATTN_ERR_UNSUPPORTED;
    if (desc->dtype != CXXATTN_F32 && desc->dtype != CXXATTN_BF16) return CXXATTN_ERR_INVALID;
    const int dev = current_device();
    if (dev < 0) return CXXATTN_ERR_CUDA;
    cxxattn_host_plan* p = new (std::nothrow) cxxattn_host_plan();
    if (p == nullptr) return CXXATTN_ERR_CUDA;
    p->desc = *desc;
    p->device = dev;
    p->chunk_b = batch_per_chunk > desc->B ? (int)desc->B : batch_per_chunk;
    const int64_t nchunks = (desc->B + p->chunk_b - 1) / p->chunk_b;
    p->nslots = nchunks < kMaxSlots ? (int)nchunks : kMaxSlots;
    p->elem = desc->dtype == CXXATTN_BF16 ? 2 : 4;
    p->chunk_elems = (size_t)p->chunk_b * desc->S * desc->H * desc->Dh;
    cxxattn_mha_desc cd = *desc;
    cd.B = p->chunk_b;
    p->ws_bytes = cxxattn_mha_bwd_workspace_bytes(&cd, 1);
    if (p->ws_bytes == 0) {
        delete p;
        return CXXATTN_ERR_UNSUPPORTED;
    }
    if (!alloc_slots(p->slots, p->nslots, 8, p->chunk_elems * p->elem,
                     (size_t)p->chunk_b * desc->H * desc->S * sizeof(float), p->ws_bytes)) {
        cxxattn_host_plan_destroy(p);
        return CXXATTN_ERR_CUDA;
    }
    *out = p;
    return CXXATTN_OK;
}

int cxxattn_mha_fwd_bwd_host(cxxattn_host_plan* plan, const void* hQ, const void* hK, const void* hV,
                             const void* hdO, void* hO, void* hdQ, void* hdK, void* hdV) {
    if (!plan || !hQ || !hK || !hV || !hdO || !hO || !hdQ || !hdK || !hdV) return CXXATTN_ERR_INVALID;
    if (current_device() != plan->device) return CXXATTN_ERR_INVALID;
    const cxxattn_mha_desc& d = plan->desc;
    const void* hin[4] = {hQ, hK, hV, hdO};
    void* hout[4] = {hO, hdQ, hdK, hdV};
    const size_t per_b = (size_t)d.S * d.H * d.Dh * plan->elem;
    int rc = CXXATTN_OK;
    int c = 0;
    for (int64_t b0 = 0; b0 < d.B && rc == CXXATTN_OK; b0 += plan->chunk_b, c++) {
        Slot& s = plan->slots[c % plan->nslots];
        const int64_t nb = d.B - b0 < plan->chunk_b ? d.B - b0 : plan->chunk_b;
        const size_t bytes = (size_t)nb * per_b, off = (size_t)b0 * per_b;
        cxxattn_mha_desc cd = d;
        cd.B = nb;
        for (int i = 0; i < 4; i++)
            if (cudaMemcpyAsync(s.buf[i], static_cast<const char*>(hin[i]) + off, bytes, cudaMemcpyHostToDevice, s.st) !=
                cudaSuccess)
                rc = CXXATTN_ERR_CUDA;
        if (rc != CXXATTN_OK) break;
        rc = cxxattn_mha_fwd(&cd, s.buf[0], s.buf[1], s.buf[2], s.buf[4], s.aux, s.st);
        if (rc != CXXATTN_OK) break;
        rc = cxxattn_mha_bwd(&cd, s.buf[0], s.buf[1], s.buf[2], s.buf[4], s.buf[3], s.aux, s.buf[5], s.buf[6],
                             s.buf[7], s.ws, plan->ws_bytes, s.st);
        if (rc != CXXATTN_OK) break;
        for (int i = 0; i < 4; i++)
            if (cudaMemcpyAsync(static_cast<char*>(hout[i]) + off, s.buf[4 + i], bytes, cudaMemcpyDeviceToHost, s.st) !=
                cudaSuccess)
                rc = CXXATTN_ERR_CUDA;
    }
    return drain(plan->slots, plan->nslots, rc);
}

void cxxattn_lin_host_plan_destroy(cxxattn_lin_host_plan* plan) {
    if (plan == nullptr) return;
    free_slots(plan->slots, plan->nslots);
    delete plan;
}

int cxxattn_lin_host_plan_create(cxxattn_lin_host_plan** out, const cxxattn_lin_desc* desc, int units_per_chunk) {
    if (out == nullptr || desc == nullptr || units_per_chunk <= 0) return CXXATTN_ERR_INVALID;
    if (desc->dtype != CXXATTN_F32 && desc->dtype != CXXATTN_BF16) return CXXATTN_ERR_INVALID;
    cxxattn_lin_desc cd = *desc;
    if (cd.B <= 0) return CXXATTN_ERR_INVALID;
    if (cd.ld_qk != 0 && cd.ld_qk != cd.D) return CXXATTN_ERR_UNSUPPORTED;  // host tensors are dense
    const int chunk_b = units_per_chunk > cd.B ? (int)cd.B : units_per_chunk;
    cd.B = chunk_b;
    // a descriptor the device-pointer entry points would refuse is refused here too
    const size_t ws = cxxattn_linattn_workspace_bytes(&cd);
    if (ws == 0 && desc->dtype == CXXATTN_F32) return CXXATTN_ERR_INVALID;
    if (desc->dtype == CXXATTN_BF16 && !linattn_tc_supported(cd) && !linattn_wide_supported(cd)) return CXXATTN_ERR_UNSUPPORTED;
    const int dev = current_device();
    if (dev < 0) return CXXATTN_ERR_CUDA;
    cxxattn_lin_host_plan* p = new (std::nothrow) cxxattn_lin_host_plan();
    if (p == nullptr) return CXXATTN_ERR_CUDA;
    p->desc = *desc;
    p->device = dev;
    p->chunk_b = chunk_b;
    const int64_t nchunks = (desc->B + chunk_b - 1) / chunk_b;
    p->nslots = nchunks < kMaxSlots ? (int)nchunks : kMaxSlots;
    p->elem = desc->dtype == CXXATTN_BF16 ? 2 : 4;
    p->ws_bytes = ws;
    const size_t width = (size_t)(desc->D > desc->E ? desc->D : desc->E);
    if (!alloc_slots(p->slots, p->nslots, 8, (size_t)chunk_b * desc->S * width * p->elem,
                     (size_t)chunk_b * desc->S * sizeof(float), ws)) {
        cxxattn_lin_host_plan_destroy(p);
        return CXXATTN_ERR_CUDA;
    }
    *out = p;
    return CXXATTN_OK;
}

int cxxattn_linattn_fwd_bwd_host(cxxattn_lin_host_plan* plan, const void* hQ, const void* hK, const void* hV,
                                 const void* hdO, void* hO, float* hden, void* hdQ, void* hdK, void* hdV) {
    if (!plan || !hQ || !hK || !hV || !hdO || !hO || !hden || !hdQ || !hdK || !hdV) return CXXATTN_ERR_INVALID;
    if (current_device() != plan->device) return CXXATTN_ERR_INVALID;
    const cxxattn_lin_desc& d = plan->desc;
    // rows of D elements: Q K dQ dK; rows of E elements: V dO O dV
    const size_t rowD = (size_t)d.S * d.D * plan->elem, rowE = (size_t)d.S * d.E * plan->elem;
    const void* hin[4] = {hQ, hK, hV, hdO};
    const size_t in_unit[4] = {rowD, rowD, rowE, rowE};
    void* hout[4] = {hO, hdQ, hdK, hdV};
    const size_t out_unit[4] = {rowE, rowD, rowD, rowE};
    int rc = CXXATTN_OK;
    int c = 0;
    for (int64_t b0 = 0; b0 < d.B && rc == CXXATTN_OK; b0 += plan->chunk_b, c++) {
        Slot& s = plan->slots[c % plan->nslots];
        const int64_t nb = d.B - b0 < plan->chunk_b ? d.B - b0 : plan->chunk_b;
        cxxattn_lin_desc cd = d;
        cd.B = nb;
        for (int i = 0; i < 4; i++)
            if (cudaMemcpyAsync(s.buf[i], static_cast<const char*>(hin[i]) + (size_t)b0 * in_unit[i], (size_t)nb * in_unit[i],
                                cudaMemcpyHostToDevice, s.st) != cudaSuccess)
                rc = CXXATTN_ERR_CUDA;
        if (rc != CXXATTN_OK) break;
        rc = cxxattn_linattn_fwd(&cd, s.buf[0], s.buf[1], s.buf[2], s.buf[4], s.aux, nullptr, s.ws, plan->ws_bytes, s.st);
        if (rc != CXXATTN_OK) break;
        rc = cxxattn_linattn_bwd(&cd, s.buf[0], s.buf[1], s.buf[2], s.buf[4], s.buf[3], s.aux, s.buf[5], s.buf[6],
                                 s.buf[7], s.ws, plan->ws_bytes, s.st);
        if (rc != CXXATTN_OK) break;
        for (int i = 0; i < 4; i++)
            if (cudaMemcpyAsync(static_cast<char*>(hout[i]) + (size_t)b0 * out_unit[i], s.buf[4 + i],
                                (size_t)nb * out_unit[i], cudaMemcpyDeviceToHost, s.st) != cudaSuccess)
                rc = CXXATTN_ERR_CUDA;
        if (cudaMemcpyAsync(hden + (size_t)b0 * d.S, s.aux, (size_t)nb * d.S * sizeof(float), cudaMemcpyDeviceToHost,
                            s.st) != cudaSuccess)
            rc = CXXATTN_ERR_CUDA;
    }
    return drain(plan->slots, plan->nslots, rc);
}

}  // extern "C"
