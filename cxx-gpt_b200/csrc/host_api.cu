// Host-buffer entry points: the caller hands over HOST pointers, the library stages the data
// through device buffers it owns.  This is the call the end-to-end benchmark times: the batch is
// cut into chunks, each chunk travels host -> device, runs forward + backward and returns
// device -> host on its own stream, so that the copies of one chunk overlap the kernels of another
// (both copy engines and the SMs stay busy).  Inputs should be page-locked for the copies to be
// asynchronous; pageable memory works but serialises.
#include "internal.cuh"
#include <vector>

using namespace cxxattn;

struct cxxattn_host_plan {
    cxxattn_mha_desc desc;      // whole problem, reference layout
    int chunk_b;                // batch items per chunk
    int nslots;
    size_t elem;                // bytes per element
    size_t chunk_elems;         // elements of one tensor of one full chunk
    size_t ws_bytes;
    struct Slot {
        cudaStream_t st;
        char* buf[8];           // Q K V dO O dQ dK dV
        float* lse;
        void* ws;
    };
    std::vector<Slot> slots;
};

extern "C" {

void cxxattn_host_plan_destroy(cxxattn_host_plan* plan) {
    if (plan == nullptr) return;
    for (auto& s : plan->slots) {
        for (char* b : s.buf) cudaFree(b);
        cudaFree(s.lse);
        cudaFree(s.ws);
        if (s.st) cudaStreamDestroy(s.st);
    }
    delete plan;
}

int cxxattn_host_plan_create(cxxattn_host_plan** out, const cxxattn_mha_desc* desc, int batch_per_chunk) {
    if (out == nullptr || desc == nullptr || batch_per_chunk <= 0) return CXXATTN_ERR_INVALID;
    if (desc->B <= 0 || desc->S <= 0 || desc->H <= 0 || desc->Dh <= 0) return CXXATTN_ERR_INVALID;
    if (desc->stride_b || desc->stride_s || desc->stride_h) return CXXATTN_ERR_UNSUPPORTED;
    if (desc->dtype != CXXATTN_F32 && desc->dtype != CXXATTN_BF16) return CXXATTN_ERR_INVALID;
    cxxattn_host_plan* p = new cxxattn_host_plan();
    p->desc = *desc;
    p->chunk_b = batch_per_chunk > desc->B ? (int)desc->B : batch_per_chunk;
    const int nchunks = (int)((desc->B + p->chunk_b - 1) / p->chunk_b);
    p->nslots = nchunks < 4 ? nchunks : 4;
    p->elem = desc->dtype == CXXATTN_BF16 ? 2 : 4;
    p->chunk_elems = (size_t)p->chunk_b * desc->S * desc->H * desc->Dh;
    cxxattn_mha_desc cd = *desc;
    cd.B = p->chunk_b;
    p->ws_bytes = cxxattn_mha_bwd_workspace_bytes(&cd, 1);
    if (p->ws_bytes == 0) {
        delete p;
        return CXXATTN_ERR_UNSUPPORTED;
    }
    p->slots.resize(p->nslots);
    for (auto& s : p->slots) {
        s = {};
    }
    for (auto& s : p->slots) {
        bool ok = cudaStreamCreateWithFlags(&s.st, cudaStreamNonBlocking) == cudaSuccess;
        for (int i = 0; i < 8 && ok; i++) ok = cudaMalloc(&s.buf[i], p->chunk_elems * p->elem) == cudaSuccess;
        ok = ok && cudaMalloc(&s.lse, (size_t)p->chunk_b * desc->H * desc->S * sizeof(float)) == cudaSuccess;
        ok = ok && cudaMalloc(&s.ws, p->ws_bytes) == cudaSuccess;
        if (!ok) {
            cxxattn_host_plan_destroy(p);
            return CXXATTN_ERR_CUDA;
        }
    }
    *out = p;
    return CXXATTN_OK;
}

int cxxattn_mha_fwd_bwd_host(cxxattn_host_plan* plan, const void* hQ, const void* hK, const void* hV,
                             const void* hdO, void* hO, void* hdQ, void* hdK, void* hdV) {
    if (!plan || !hQ || !hK || !hV || !hdO || !hO || !hdQ || !hdK || !hdV) return CXXATTN_ERR_INVALID;
    const cxxattn_mha_desc& d = plan->desc;
    const void* hin[4] = {hQ, hK, hV, hdO};
    void* hout[4] = {hO, hdQ, hdK, hdV};
    const size_t per_b = (size_t)d.S * d.H * d.Dh * plan->elem;
    int rc = CXXATTN_OK;
    int c = 0;
    for (int64_t b0 = 0; b0 < d.B && rc == CXXATTN_OK; b0 += plan->chunk_b, c++) {
        auto& s = plan->slots[c % plan->nslots];
        const int64_t nb = d.B - b0 < plan->chunk_b ? d.B - b0 : plan->chunk_b;
        const size_t bytes = (size_t)nb * per_b, off = (size_t)b0 * per_b;
        cxxattn_mha_desc cd = d;
        cd.B = nb;
        for (int i = 0; i < 4; i++)
            if (cudaMemcpyAsync(s.buf[i], static_cast<const char*>(hin[i]) + off, bytes, cudaMemcpyHostToDevice, s.st) !=
                cudaSuccess)
                rc = CXXATTN_ERR_CUDA;
        if (rc != CXXATTN_OK) break;
        rc = cxxattn_mha_fwd(&cd, s.buf[0], s.buf[1], s.buf[2], s.buf[4], s.lse, s.st);
        if (rc != CXXATTN_OK) break;
        rc = cxxattn_mha_bwd(&cd, s.buf[0], s.buf[1], s.buf[2], s.buf[4], s.buf[3], s.lse, s.buf[5], s.buf[6],
                             s.buf[7], s.ws, plan->ws_bytes, s.st);
        if (rc != CXXATTN_OK) break;
        for (int i = 0; i < 4; i++)
            if (cudaMemcpyAsync(static_cast<char*>(hout[i]) + off, s.buf[4 + i], bytes, cudaMemcpyDeviceToHost, s.st) !=
                cudaSuccess)
                rc = CXXATTN_ERR_CUDA;
    }
    for (auto& s : plan->slots)
        if (cudaStreamSynchronize(s.st) != cudaSuccess && rc == CXXATTN_OK) rc = CXXATTN_ERR_CUDA;
    return rc;
}

}  // extern "C"
