// The multi-GPU host driver: the (batch x head) space of one attention call split over the GPUs of a box,
// one process per GPU, with NCCL used only to all-gather the outputs (no counterpart in the reference,
// which runs on one GPU; every (batch, head) pair of its kernels is independent, src/hip_kernels.cpp:269-277,
// which is what makes the split exact).
//
// Batches are dealt to the ranks chunk by chunk: with `chunks` chunks of k = B / (world * chunks) batches per
// rank, chunk c covers global batches [c*world*k, (c+1)*world*k) and rank r owns the r-th run of k batches in
// it.  In the [B*S][E] output that makes every chunk one contiguous [world][k*S*E] block with the rank's own
// part at offset rank * k*S*E: exactly the in-place form of ncclAllGather (sendbuff = recvbuff + rank * count),
// so no staging copy is needed.  Per chunk: the attention kernels on the caller's stream, an event, then the
// all-gather of that chunk on a communication stream of the highest priority, so that NCCL's thread blocks
// are placed as soon as blocks of the next chunk's attention kernel retire, and the transfer of chunk c
// overlaps the arithmetic of chunk c + 1.  The kernels read local memory only.
//
// Second transport (gather = HIPGPT_GATHER_PEER_STORES): NCCL's thread blocks are large and wait for attention blocks
// to retire before they find room, and the measured time of the NCCL form is close to compute + gather.  Here every
// rank maps every other rank's output buffer (inter-process memory handles, exchanged once through the
// communicator), and after a chunk's kernels a copy kernel of 128-thread blocks without shared memory
// (shard_push.cu) stores the chunk into the peers' buffers with plain stores over NVLink; those blocks fit beside two
// resident attention blocks on every SM.  No kernel waits for another GPU: a four-byte-per-rank collective on the
// communication stream before the first copy (every rank has reached this call on its stream, so its buffer may be
// written) and after the last one (every rank's copies have completed, which for a kernel means performed) orders
// the ranks.
// Third transport (gather = HIPGPT_GATHER_PEER_COPIES): the same mapped buffers and the same ordering, but the data is
// moved by copy engines: one cudaMemcpyAsync per peer and chunk, each on a stream of its peer, so that no SM and no issue
// slot is taken from the attention kernels.  gather = HIPGPT_GATHER_PEER_BOTH serves some peers one way and the others the
// other way at the same time (HIPGPT_GATHER_COPY_PEERS overrides how many go to the copy engines).
//
// NCCL is loaded at run time (dlopen of libnccl.so.2: in a torch process that is the copy torch already
// loaded), so the single-GPU library has no link dependency on it.
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "attn_common.cuh"

namespace hipgpt {
namespace {

// the handful of NCCL declarations used here (nccl.h, ABI-stable since 2.x)
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
constexpr int ncclChar = 0;

struct Nccl {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GetVersion)(int *) = nullptr;
};

Nccl *nccl()
{
    static Nccl api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char *override_path = getenv("HIPGPT_NCCL_LIB");
        void *h = dlopen(override_path && override_path[0] ? override_path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return;
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(h, "ncclAllGather"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
        api.GetVersion = reinterpret_cast<decltype(api.GetVersion)>(dlsym(h, "ncclGetVersion"));
        if (api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.GetErrorString) api.handle = h;
    });
    return api.handle ? &api : nullptr;
}

int nccl_fail(Nccl *n, ncclResult_t r, const char *what) { return fail(HIPGPT_ERR_CUDA, "%s: %s", what, n->GetErrorString(r)); }

int cuda_fail(cudaError_t e, const char *what) { return fail(HIPGPT_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e)); }

}  // namespace
}  // namespace hipgpt

using namespace hipgpt;

struct hipgpt_shard_ctx {
    int rank = 0, world = 1, device = 0;
    ncclComm_t comm = nullptr;
    cudaStream_t comm_stream = nullptr;
    static constexpr int kMaxChunks = 64;
    cudaEvent_t computed[kMaxChunks] = {};      // chunk c's attention kernels have been enqueued and will have finished
    cudaEvent_t gathered = nullptr;             // the last all-gather has finished
    cudaEvent_t entered = nullptr;              // the caller's stream has reached the call
    // peer-store transport
    static constexpr int kMaxPeers = 8;
    uint8_t *own_out = nullptr;                 // this rank's output buffer (hipgpt_shard_output_buffer)
    size_t own_bytes = 0;
    uint8_t *peer_out[kMaxPeers] = {};          // the same buffer of every rank as mapped here; [rank] = own_out
    int *sync_words = nullptr;                  // [world] ints on the device: the ordering collective's operand
    cudaStream_t peer_stream[kMaxPeers] = {};   // copy-engine transport: one stream per peer, so that the copies to different peers run side by side
    cudaEvent_t peer_done[kMaxPeers] = {};
};

extern "C" {

int hipgpt_shard_chunk_range(int B, int world, int rank, int chunks, int chunk, int *b_begin, int *b_end)
{
    if (B < 0 || world <= 0 || rank < 0 || rank >= world || chunks <= 0 || chunk < 0 || chunk >= chunks)
        return fail(HIPGPT_ERR_BAD_ARG, "bad request: B=%d world=%d rank=%d chunks=%d chunk=%d", B, world, rank, chunks, chunk);
    if (!b_begin || !b_end) return fail(HIPGPT_ERR_NULL, "b_begin and b_end must not be NULL");
    if (B % (world * chunks) != 0) return fail(HIPGPT_ERR_BAD_ARG, "B=%d is not a multiple of world * chunks = %d", B, world * chunks);
    const int k = B / (world * chunks);
    *b_begin = chunk * world * k + rank * k;
    *b_end = *b_begin + k;
    return HIPGPT_OK;
}

// 128 bytes that every rank must pass to hipgpt_shard_create; rank 0 makes them and sends them to the others
// by whatever means the job has (a torch.distributed broadcast, a file, a socket).
int hipgpt_shard_unique_id(void *id128)
{
    if (!id128) return fail(HIPGPT_ERR_NULL, "id128 must not be NULL");
    Nccl *n = nccl();
    if (!n) return fail(HIPGPT_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded: %s", dlerror());
    ncclUniqueId id;
    const ncclResult_t r = n->GetUniqueId(&id);
    if (r != 0) return nccl_fail(n, r, "ncclGetUniqueId");
    memcpy(id128, &id, sizeof(id));
    return HIPGPT_OK;
}

// Collective: every rank of the job calls it, each with its own GPU current.
int hipgpt_shard_create(hipgpt_shard_ctx **out, const void *id128, int rank, int world)
{
    if (!out || !id128) return fail(HIPGPT_ERR_NULL, "out and id128 must not be NULL");
    if (world <= 0 || rank < 0 || rank >= world) return fail(HIPGPT_ERR_BAD_ARG, "bad rank %d of %d", rank, world);
    hipgpt_shard_ctx *c = new hipgpt_shard_ctx;
    c->rank = rank;
    c->world = world;
    cudaError_t e = cudaGetDevice(&c->device);
    int lo = 0, hi = 0;
    if (e == cudaSuccess) e = cudaDeviceGetStreamPriorityRange(&lo, &hi);     // hi is the numerically smallest, i.e. most urgent
    if (e == cudaSuccess) e = cudaStreamCreateWithPriority(&c->comm_stream, cudaStreamNonBlocking, hi);
    for (int i = 0; i < hipgpt_shard_ctx::kMaxChunks && e == cudaSuccess; ++i) e = cudaEventCreateWithFlags(&c->computed[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->gathered, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->entered, cudaEventDisableTiming);
    for (int p = 0; p < world && p < hipgpt_shard_ctx::kMaxPeers && e == cudaSuccess; ++p) {
        if (p == rank) continue;
        e = cudaStreamCreateWithPriority(&c->peer_stream[p], cudaStreamNonBlocking, hi);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->peer_done[p], cudaEventDisableTiming);
    }
    if (e == cudaSuccess) e = cudaMalloc(&c->sync_words, sizeof(int) * (size_t)(world > 0 ? world : 1));
    if (e == cudaSuccess) e = cudaMemset(c->sync_words, 0, sizeof(int) * (size_t)world);
    if (e != cudaSuccess) {
        hipgpt_shard_destroy(c);
        return fail(HIPGPT_ERR_CUDA, "stream or event creation: %s", cudaGetErrorString(e));
    }
    if (world > 1) {
        Nccl *n = nccl();
        if (!n) { hipgpt_shard_destroy(c); return fail(HIPGPT_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded"); }
        ncclUniqueId id;
        memcpy(&id, id128, sizeof(id));
        const ncclResult_t r = n->CommInitRank(&c->comm, world, id, rank);
        if (r != 0) { hipgpt_shard_destroy(c); return nccl_fail(n, r, "ncclCommInitRank"); }
    }
    *out = c;
    return HIPGPT_OK;
}

// Every rank has passed this point on its communication stream (a collective of four bytes per rank), and the host has waited for it.
static int ranks_meet(hipgpt_shard_ctx *c)
{
    if (c->world > 1 && c->comm) {
        Nccl *n = nccl();
        const ncclResult_t r = n->AllGather(c->sync_words + c->rank, c->sync_words, sizeof(int), ncclChar, c->comm, c->comm_stream);
        if (r != 0) return nccl_fail(n, r, "ncclAllGather (ordering)");
    }
    const cudaError_t e = cudaStreamSynchronize(c->comm_stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamSynchronize");
    return HIPGPT_OK;
}

// Unmaps the peers' buffers, waits until every rank has done so, frees this rank's.
static int release_output_buffer(hipgpt_shard_ctx *c)
{
    if (!c->own_out) return HIPGPT_OK;
    cudaDeviceSynchronize();
    for (int p = 0; p < c->world && p < hipgpt_shard_ctx::kMaxPeers; ++p)
        if (p != c->rank && c->peer_out[p]) cudaIpcCloseMemHandle(c->peer_out[p]);
    const int rc = ranks_meet(c);
    cudaFree(c->own_out);
    c->own_out = nullptr;
    c->own_bytes = 0;
    for (auto &p : c->peer_out) p = nullptr;
    return rc;
}

int hipgpt_shard_output_buffer(hipgpt_shard_ctx *c, size_t bytes, void **d_out)
{
    if (!c || !d_out) return fail(HIPGPT_ERR_NULL, "context and d_out must not be NULL");
    if (c->world > hipgpt_shard_ctx::kMaxPeers) return fail(HIPGPT_ERR_UNSUPPORTED, "the peer-store transport takes at most %d ranks", hipgpt_shard_ctx::kMaxPeers);
    if (bytes == 0) return fail(HIPGPT_ERR_BAD_ARG, "an output buffer of 0 bytes");
    int rc = release_output_buffer(c);
    if (rc != HIPGPT_OK) return rc;
    cudaError_t e = cudaMalloc(&c->own_out, bytes);
    if (e != cudaSuccess) { c->own_out = nullptr; return cuda_fail(e, "cudaMalloc of the output buffer"); }
    c->own_bytes = bytes;
    c->peer_out[c->rank] = c->own_out;
    if (c->world > 1) {
        // the handles travel through the communicator: [world] handles on the device, all-gathered in place
        Nccl *n = nccl();
        cudaIpcMemHandle_t mine, all[hipgpt_shard_ctx::kMaxPeers];
        uint8_t *d_handles = nullptr;
        e = cudaIpcGetMemHandle(&mine, c->own_out);
        if (e == cudaSuccess) e = cudaMalloc(&d_handles, sizeof(mine) * (size_t)c->world);
        if (e == cudaSuccess) e = cudaMemcpyAsync(d_handles + sizeof(mine) * (size_t)c->rank, &mine, sizeof(mine), cudaMemcpyHostToDevice, c->comm_stream);
        if (e != cudaSuccess) { cudaFree(d_handles); return cuda_fail(e, "inter-process handle of the output buffer"); }
        const ncclResult_t r = n->AllGather(d_handles + sizeof(mine) * (size_t)c->rank, d_handles, sizeof(mine), ncclChar, c->comm, c->comm_stream);
        if (r != 0) { cudaFree(d_handles); return nccl_fail(n, r, "ncclAllGather (handles)"); }
        e = cudaMemcpyAsync(all, d_handles, sizeof(mine) * (size_t)c->world, cudaMemcpyDeviceToHost, c->comm_stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->comm_stream);
        cudaFree(d_handles);
        if (e != cudaSuccess) return cuda_fail(e, "exchange of the handles");
        for (int p = 0; p < c->world; ++p) {
            if (p == c->rank) continue;
            void *mapped = nullptr;
            e = cudaIpcOpenMemHandle(&mapped, all[p], cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) return cuda_fail(e, "cudaIpcOpenMemHandle of a peer's output buffer");
            c->peer_out[p] = static_cast<uint8_t *>(mapped);
        }
        rc = ranks_meet(c);                      // every rank has mapped every buffer before any of them is used
        if (rc != HIPGPT_OK) return rc;
    }
    *d_out = c->own_out;
    return HIPGPT_OK;
}

void hipgpt_shard_destroy(hipgpt_shard_ctx *c)
{
    if (!c) return;
    release_output_buffer(c);
    if (c->sync_words) cudaFree(c->sync_words);
    for (auto &ps : c->peer_stream) if (ps) cudaStreamDestroy(ps);
    for (auto &pe : c->peer_done) if (pe) cudaEventDestroy(pe);
    if (c->entered) cudaEventDestroy(c->entered);
    if (c->comm) nccl()->CommDestroy(c->comm);
    for (cudaEvent_t ev : c->computed) if (ev) cudaEventDestroy(ev);
    if (c->gathered) cudaEventDestroy(c->gathered);
    if (c->comm_stream) cudaStreamDestroy(c->comm_stream);
    delete c;
}

// d_q, d_k, d_v: THIS RANK'S batches only, chunk after chunk ([chunks][k][S][E], k = B / (world * chunks)): the
// global batches hipgpt_shard_chunk_range names.  d_out: the whole [B*S][E] output; on return (in stream order on
// `stream`) every batch of it is valid on every rank when gather != 0, this rank's batches only otherwise.
// elem_bytes 4: fp32 (hipgpt_mha_forward); 2: bf16 (hipgpt_mha_forward_bf16, head_dim 64).
int hipgpt_mha_forward_sharded(hipgpt_shard_ctx *c, const void *d_q, const void *d_k, const void *d_v, void *d_out,
                               int B, int S, int E, int H, int causal, int elem_bytes, int chunks, int gather, void *stream)
{
    if (!c) return fail(HIPGPT_ERR_NULL, "context must not be NULL");
    if (elem_bytes != 4 && elem_bytes != 2) return fail(HIPGPT_ERR_BAD_ARG, "elem_bytes %d is neither 4 (fp32) nor 2 (bf16)", elem_bytes);
    if (B < 0 || S < 0 || E < 0 || chunks <= 0 || chunks > hipgpt_shard_ctx::kMaxChunks)
        return fail(HIPGPT_ERR_BAD_ARG, "bad size: B=%d S=%d E=%d chunks=%d (at most %d)", B, S, E, chunks, hipgpt_shard_ctx::kMaxChunks);
    if (B % (c->world * chunks) != 0)
        return fail(HIPGPT_ERR_BAD_ARG, "B=%d is not a multiple of world * chunks = %d", B, c->world * chunks);
    if (B == 0 || S == 0 || E == 0) return HIPGPT_OK;
    if (!d_q || !d_k || !d_v || !d_out) return fail(HIPGPT_ERR_NULL, "q, k, v and out must not be NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int k = B / (c->world * chunks);
    const size_t batch = (size_t)S * E * elem_bytes;             // bytes of one batch item of a plane
    if (gather < 0 || gather > HIPGPT_GATHER_PEER_BOTH) return fail(HIPGPT_ERR_BAD_ARG, "gather = %d is none of 0, 1, 2, 3, 4", gather);
    const bool comm = gather && c->world > 1;
    const bool push = comm && gather >= HIPGPT_GATHER_PEER_STORES;            // any transport into the peers' mapped buffers
    // peers (rank + 1 .. rank + n_copy) are served by copy engines, the others by the copy kernel's stores
    int n_copy = 0;
    if (comm && gather == HIPGPT_GATHER_PEER_COPIES) n_copy = c->world - 1;
    if (comm && gather == HIPGPT_GATHER_PEER_BOTH) {
        n_copy = ((c->world - 1) * 3 + 3) / 7;       // the two transports' rates beside the kernels measured about 3 : 4
        if (const char *env = getenv("HIPGPT_GATHER_COPY_PEERS")) n_copy = atoi(env);
        if (n_copy < 0) n_copy = 0;
        if (n_copy > c->world - 1) n_copy = c->world - 1;
    }
    const bool dma = n_copy > 0;
    const bool stores = push && n_copy < c->world - 1;
    Nccl *n = comm ? nccl() : nullptr;
    if (push) {
        const uint8_t *o = static_cast<const uint8_t *>(d_out);
        const size_t need = (size_t)B * batch;
        if (!c->own_out || o < c->own_out || o + need > c->own_out + c->own_bytes)
            return fail(HIPGPT_ERR_BAD_ARG, "gather = 2, 3 and 4 need d_out inside the buffer of hipgpt_shard_output_buffer (%zu bytes needed)", need);
        if (((size_t)k * batch) & 15) return fail(HIPGPT_ERR_BAD_ARG, "a rank's chunk of %zu bytes is not a multiple of 16", (size_t)k * batch);
        // no rank writes into a peer that has not reached this call on its stream
        cudaError_t e = cudaEventRecord(c->entered, st);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(c->comm_stream, c->entered, 0);
        if (e != cudaSuccess) return cuda_fail(e, "event hand-off");
        const ncclResult_t r = n->AllGather(c->sync_words + c->rank, c->sync_words, sizeof(int), ncclChar, c->comm, c->comm_stream);
        if (r != 0) return nccl_fail(n, r, "ncclAllGather (ordering)");
        if (dma) {
            // the per-peer copy streams start behind that collective
            e = cudaEventRecord(c->entered, c->comm_stream);
            for (int i = 1; i <= n_copy && e == cudaSuccess; ++i) e = cudaStreamWaitEvent(c->peer_stream[(c->rank + i) % c->world], c->entered, 0);
            if (e != cudaSuccess) return cuda_fail(e, "event hand-off");
        }
    }
    const uint8_t *q = static_cast<const uint8_t *>(d_q), *kk = static_cast<const uint8_t *>(d_k), *v = static_cast<const uint8_t *>(d_v);
    uint8_t *out = static_cast<uint8_t *>(d_out);
    for (int ch = 0; ch < chunks; ++ch) {
        const size_t in_off = (size_t)ch * k * batch;                          // this rank's chunk ch of the local planes
        uint8_t *block = out + (size_t)ch * c->world * k * batch;              // chunk ch of the output: [world][k batches]
        uint8_t *mine = block + (size_t)c->rank * k * batch;
        const int rc = elem_bytes == 4
            ? hipgpt_mha_forward(reinterpret_cast<const float *>(q + in_off), reinterpret_cast<const float *>(kk + in_off),
                                 reinterpret_cast<const float *>(v + in_off), reinterpret_cast<float *>(mine), nullptr, k, S, E, H, causal, st)
            : hipgpt_mha_forward_bf16(q + in_off, kk + in_off, v + in_off, mine, k, S, E, H, causal, st);
        if (rc != HIPGPT_OK) return rc;
        if (!comm) continue;
        cudaError_t e = cudaEventRecord(c->computed[ch], st);
        if (e == cudaSuccess && (!push || stores)) e = cudaStreamWaitEvent(c->comm_stream, c->computed[ch], 0);
        if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "event hand-off: %s", cudaGetErrorString(e));
        if (push) {
            const size_t off = (size_t)(mine - c->own_out);
            // one copy per copy-engine peer and chunk, each on its peer's stream: no SM is used
            for (int i = 1; i <= n_copy && e == cudaSuccess; ++i) {
                const int p = (c->rank + i) % c->world;
                e = cudaStreamWaitEvent(c->peer_stream[p], c->computed[ch], 0);
                if (e == cudaSuccess) e = cudaMemcpyAsync(c->peer_out[p] + off, mine, (size_t)k * batch, cudaMemcpyDeviceToDevice, c->peer_stream[p]);
            }
            if (e != cudaSuccess) return cuda_fail(e, "peer copy");
            if (stores) {
                void *dst[hipgpt_shard_ctx::kMaxPeers];
                int nd = 0;
                for (int i = n_copy + 1; i < c->world; ++i) dst[nd++] = c->peer_out[(c->rank + i) % c->world] + off;
                const int prc = launch_shard_push(mine, dst, nd, (size_t)k * batch, c->comm_stream);
                if (prc != HIPGPT_OK) return prc;
            }
            continue;
        }
        const ncclResult_t r = n->AllGather(mine, block, (size_t)k * batch, ncclChar, c->comm, c->comm_stream);
        if (r != 0) return nccl_fail(n, r, "ncclAllGather");
    }
    if (dma) {
        cudaError_t e = cudaSuccess;
        for (int i = 1; i <= n_copy && e == cudaSuccess; ++i) {
            const int p = (c->rank + i) % c->world;
            e = cudaEventRecord(c->peer_done[p], c->peer_stream[p]);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(c->comm_stream, c->peer_done[p], 0);
        }
        if (e != cudaSuccess) return cuda_fail(e, "event hand-off");
    }
    if (push) {
        // every rank's copies have completed (a kernel, or a copy, that has completed has performed its stores)
        const ncclResult_t r = n->AllGather(c->sync_words + c->rank, c->sync_words, sizeof(int), ncclChar, c->comm, c->comm_stream);
        if (r != 0) return nccl_fail(n, r, "ncclAllGather (ordering)");
    }
    if (comm) {
        cudaError_t e = cudaEventRecord(c->gathered, c->comm_stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(st, c->gathered, 0);    // later work on the caller's stream sees the whole output
        if (e != cudaSuccess) return fail(HIPGPT_ERR_CUDA, "event hand-off: %s", cudaGetErrorString(e));
    }
    return HIPGPT_OK;
}

int hipgpt_shard_nccl_version(void)
{
    Nccl *n = nccl();
    int v = 0;
    if (!n || !n->GetVersion || n->GetVersion(&v) != 0) return 0;
    return v;
}

}  // extern "C"
