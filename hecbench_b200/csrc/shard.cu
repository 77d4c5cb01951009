// Output-feature sharding of one layer over the GPUs of a node, for a C or C++
// host that drives all GPUs from ONE process (no counterpart in the reference
// tree; its only multi-GPU code is the NCCL sample ccl-cuda/main.cu:83-117,
// whose create / collective / destroy sequence the optional NCCL part follows).
//
// A context owns, per GPU ("rank"): a stream, `slots` gathered buffers in both
// forms of include/hq.h - packet vectors for the low-latency gather of the
// batch-1 NF4 GEMV and fp16 buffers [world][rows][n_local] with flag words for
// the copy + flag gather - the device-resident pointer tables the kernels
// take, the per-rank sync words and a status word.  Peer access is enabled
// between every pair of GPUs, so a buffer of one GPU is addressed by the
// kernels of another through its ordinary pointer.
//
// The host calls the per-rank entries for rank 0 .. world-1 in turn; every
// call is asynchronous on that rank's stream.  A kernel that waits for another
// rank's data does so with a bounded poll, and the other rank's kernel runs on
// another GPU, so the order in which one host thread issues the launches does
// not matter as long as all ranks are issued within the poll limit (about a
// second).
#include <dlfcn.h>
#include <nccl.h>

#include <new>
#include <vector>

#include "hq_common.cuh"

struct hq_shard_ctx {
  int world = 0, rows = 1, slots = 0;
  long long n_local = 0;
  std::vector<int> devices;
  std::vector<cudaStream_t> streams;
  std::vector<unsigned char*> packets;   // per rank: [slots][world * n_local] packets
  std::vector<unsigned char*> gathered;  // per rank: 256 B of flags, then [slots][world][rows][n_local] fp16
  std::vector<unsigned char*> tables;    // per rank: pointer tables + sync words + status
  // optional NCCL
  void* nccl_lib = nullptr;
  std::vector<ncclComm_t> comms;
  ncclResult_t (*pGroupStart)() = nullptr;
  ncclResult_t (*pGroupEnd)() = nullptr;
  ncclResult_t (*pAllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t,
                             cudaStream_t) = nullptr;
  ncclResult_t (*pCommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*pCommDestroy)(ncclComm_t) = nullptr;
};

namespace hq {
namespace {

// Layout of a rank's table block (device memory, 8-byte units):
//   [slots][world] packet-vector pointers | [world] gathered-data pointers |
//   [world] flag-array pointers | 2 + 2 sync words | status word
struct TableLayout {
  size_t peer_ll, peer_data, peer_flags, sync_ll, sync_pub, status, bytes;
};
TableLayout table_layout(int world, int slots) {
  TableLayout t;
  t.peer_ll = 0;
  t.peer_data = t.peer_ll + (size_t)slots * world * 8;
  t.peer_flags = t.peer_data + (size_t)world * 8;
  t.sync_ll = t.peer_flags + (size_t)world * 8;
  t.sync_pub = t.sync_ll + 8;
  t.status = t.sync_pub + 8;
  t.bytes = t.status + 8;
  return t;
}

struct DeviceGuard {
  int prev = -1;
  cudaError_t err;
  explicit DeviceGuard(int dev) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess) err = cudaSetDevice(dev);
  }
  ~DeviceGuard() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

bool rank_ok(const hq_shard_ctx* c, int rank, int slot) {
  return c != nullptr && rank >= 0 && rank < c->world && slot >= 0 && slot < c->slots;
}

}  // namespace
}  // namespace hq

extern "C" {

int hq_shard_layout(int world, int rows, long long n_local, int slots, int rank, int slot,
                    long long* packet_index, long long* slice_index, long long* slot_elems) {
  if (world < 1 || world > 32 || rows < 1 || n_local < 1 || slots < 1) return HQ_ERR_BAD_SHAPE;
  if (rank < 0 || rank >= world || slot < 0 || slot >= slots) return HQ_ERR_BAD_SHAPE;
  const long long per_slot = (long long)world * rows * n_local;
  if (slot_elems) *slot_elems = per_slot;
  // packets exist for mat-vec outputs only (rows == 1): rank r's results start at r * n_local
  if (packet_index) *packet_index = (long long)slot * world * n_local + (long long)rank * n_local;
  if (slice_index) *slice_index = (long long)slot * per_slot + (long long)rank * rows * n_local;
  return HQ_OK;
}

void hq_shard_destroy(hq_shard_ctx* c) {
  using namespace hq;
  if (c == nullptr) return;
  for (size_t r = 0; r < c->comms.size(); r++)
    if (c->comms[r] != nullptr && c->pCommDestroy) c->pCommDestroy(c->comms[r]);
  for (int r = 0; r < (int)c->devices.size(); r++) {
    DeviceGuard g(c->devices[r]);
    if (r < (int)c->streams.size() && c->streams[r]) {
      cudaStreamSynchronize(c->streams[r]);
      cudaStreamDestroy(c->streams[r]);
    }
    if (r < (int)c->packets.size()) cudaFree(c->packets[r]);
    if (r < (int)c->gathered.size()) cudaFree(c->gathered[r]);
    if (r < (int)c->tables.size()) cudaFree(c->tables[r]);
  }
  if (c->nccl_lib) dlclose(c->nccl_lib);
  delete c;
}

int hq_shard_create(hq_shard_ctx** out, const int* devices, int world, long long n_local, int rows,
                    int slots, int flags) {
  using namespace hq;
  if (!out || !devices) return HQ_ERR_NULL_POINTER;
  *out = nullptr;
  if (world < 1 || world > 32 || n_local < 1 || rows < 1 || rows > 128 || slots < 2)
    return HQ_ERR_BAD_SHAPE;  // a chain of gathers alternates between at least two buffers
  hq_shard_ctx* c = new (std::nothrow) hq_shard_ctx();
  if (!c) return HQ_ERR_CUDA;
  c->world = world;
  c->rows = rows;
  c->slots = slots;
  c->n_local = n_local;
  c->devices.assign(devices, devices + world);
  c->streams.assign(world, nullptr);
  c->packets.assign(world, nullptr);
  c->gathered.assign(world, nullptr);
  c->tables.assign(world, nullptr);
  const TableLayout tl = table_layout(world, slots);
  const size_t slot_elems = (size_t)world * rows * n_local;
  const size_t packet_bytes = (size_t)slots * world * n_local * 8;
  const size_t gathered_bytes = 256 + (size_t)slots * slot_elems * 2;
  auto fail = [&](cudaError_t e) {
    const int st = e == cudaSuccess ? HQ_ERR_UNSUPPORTED : cuda_status(e);
    hq_shard_destroy(c);
    return st;
  };
  for (int r = 0; r < world; r++) {
    DeviceGuard g(devices[r]);
    if (g.err != cudaSuccess) return fail(g.err);
    for (int p = 0; p < world; p++) {
      if (p == r || devices[p] == devices[r]) continue;
      int can = 0;
      cudaError_t e = cudaDeviceCanAccessPeer(&can, devices[r], devices[p]);
      if (e != cudaSuccess) return fail(e);
      if (!can) return fail(cudaSuccess);
      e = cudaDeviceEnablePeerAccess(devices[p], 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
      else if (e != cudaSuccess) return fail(e);
    }
    cudaError_t e = cudaStreamCreateWithFlags(&c->streams[r], cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->packets[r], packet_bytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->gathered[r], gathered_bytes);
    if (e == cudaSuccess) e = cudaMalloc((void**)&c->tables[r], tl.bytes);
    if (e == cudaSuccess) e = cudaMemset(c->packets[r], 0, packet_bytes);
    if (e == cudaSuccess) e = cudaMemset(c->gathered[r], 0, gathered_bytes);
    if (e == cudaSuccess) e = cudaMemset(c->tables[r], 0, tl.bytes);
    if (e != cudaSuccess) return fail(e);
  }
  // pointer tables (the same on every rank)
  std::vector<unsigned char> host(tl.bytes, 0);
  auto put = [&](size_t off, const void* p) { memcpy(host.data() + off, &p, 8); };
  for (int s = 0; s < slots; s++)
    for (int p = 0; p < world; p++)
      put(tl.peer_ll + ((size_t)s * world + p) * 8,
          c->packets[p] + (size_t)s * world * n_local * 8);
  for (int p = 0; p < world; p++) {
    put(tl.peer_data + (size_t)p * 8, c->gathered[p] + 256);
    put(tl.peer_flags + (size_t)p * 8, c->gathered[p]);
  }
  for (int r = 0; r < world; r++) {
    DeviceGuard g(devices[r]);
    cudaError_t e = cudaMemcpy(c->tables[r], host.data(), tl.bytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail(e);
  }
  if (flags & HQ_SHARD_NCCL) {
    // the communicators of ccl-cuda/main.cu:83-91, through a library loaded on demand
    c->nccl_lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!c->nccl_lib) return fail(cudaSuccess);
    auto init_all = (ncclResult_t(*)(ncclComm_t*, int, const int*))dlsym(c->nccl_lib, "ncclCommInitAll");
    c->pGroupStart = (ncclResult_t(*)())dlsym(c->nccl_lib, "ncclGroupStart");
    c->pGroupEnd = (ncclResult_t(*)())dlsym(c->nccl_lib, "ncclGroupEnd");
    c->pAllGather = (ncclResult_t(*)(const void*, void*, size_t, ncclDataType_t, ncclComm_t,
                                     cudaStream_t))dlsym(c->nccl_lib, "ncclAllGather");
    c->pCommAbort = (ncclResult_t(*)(ncclComm_t))dlsym(c->nccl_lib, "ncclCommAbort");
    c->pCommDestroy = (ncclResult_t(*)(ncclComm_t))dlsym(c->nccl_lib, "ncclCommDestroy");
    if (!init_all || !c->pGroupStart || !c->pGroupEnd || !c->pAllGather || !c->pCommAbort ||
        !c->pCommDestroy)
      return fail(cudaSuccess);
    c->comms.assign(world, nullptr);
    if (init_all(c->comms.data(), world, devices) != ncclSuccess) {
      c->comms.clear();
      hq_shard_destroy(c);
      return HQ_ERR_NCCL;
    }
  }
  *out = c;
  return HQ_OK;
}

hq_stream_t hq_shard_stream(hq_shard_ctx* c, int rank) {
  return hq::rank_ok(c, rank, 0) ? (hq_stream_t)c->streams[rank] : nullptr;
}

void* hq_shard_local_slice(hq_shard_ctx* c, int rank, int slot) {
  if (!hq::rank_ok(c, rank, slot)) return nullptr;
  long long idx = 0;
  hq_shard_layout(c->world, c->rows, c->n_local, c->slots, rank, slot, nullptr, &idx, nullptr);
  return c->gathered[rank] + 256 + (size_t)idx * 2;
}

const void* hq_shard_gathered(hq_shard_ctx* c, int rank, int slot) {
  if (!hq::rank_ok(c, rank, slot)) return nullptr;
  return c->gathered[rank] + 256 + (size_t)slot * c->world * c->rows * c->n_local * 2;
}

int hq_shard_nf4_gemv(hq_shard_ctx* c, int rank, int slot, const void* A_half, int a_slot,
                      long long a_stride, const uint8_t* B, const float* absmax,
                      const float* lut16, int K, int blocksize, int flags) {
  using namespace hq;
  if (!rank_ok(c, rank, slot) || c->rows != 1) return HQ_ERR_BAD_SHAPE;
  if (A_half == nullptr && !rank_ok(c, rank, a_slot)) return HQ_ERR_BAD_SHAPE;
  if (c->n_local > 0x7fffffffLL) return HQ_ERR_TOO_LARGE;
  const TableLayout tl = table_layout(c->world, c->slots);
  DeviceGuard g(c->devices[rank]);
  if (g.err != cudaSuccess) return cuda_status(g.err);
  const hq_ll_packet* a_ll = nullptr;
  if (A_half == nullptr)
    a_ll = reinterpret_cast<const hq_ll_packet*>(c->packets[rank] +
                                                 (size_t)a_slot * c->world * c->n_local * 8);
  unsigned char* tab = c->tables[rank];
  return hq_nf4_gemv_f16_ll(
      A_half, a_ll, a_stride, B, absmax, lut16, nullptr, (int)c->n_local, K, blocksize, flags,
      reinterpret_cast<hq_ll_packet* const*>(tab + tl.peer_ll + (size_t)slot * c->world * 8),
      (long long)rank * c->n_local, reinterpret_cast<unsigned*>(tab + tl.sync_ll), c->world, rank,
      0, reinterpret_cast<int*>(tab + tl.status), (hq_stream_t)c->streams[rank]);
}

int hq_shard_unpack(hq_shard_ctx* c, int rank, int slot, void* out_half) {
  using namespace hq;
  if (!rank_ok(c, rank, slot) || c->rows != 1) return HQ_ERR_BAD_SHAPE;
  const TableLayout tl = table_layout(c->world, c->slots);
  DeviceGuard g(c->devices[rank]);
  if (g.err != cudaSuccess) return cuda_status(g.err);
  unsigned char* tab = c->tables[rank];
  return hq_ll_unpack(
      reinterpret_cast<const hq_ll_packet*>(c->packets[rank] +
                                            (size_t)slot * c->world * c->n_local * 8),
      (long long)c->world * c->n_local, out_half, reinterpret_cast<unsigned*>(tab + tl.sync_ll), 0,
      reinterpret_cast<int*>(tab + tl.status), (hq_stream_t)c->streams[rank]);
}

int hq_shard_publish(hq_shard_ctx* c, int rank, int slot) {
  using namespace hq;
  if (!rank_ok(c, rank, slot)) return HQ_ERR_BAD_SHAPE;
  const long long slice = (long long)c->rows * c->n_local;
  if (slice > 0x7fffffffLL) return HQ_ERR_TOO_LARGE;
  const TableLayout tl = table_layout(c->world, c->slots);
  DeviceGuard g(c->devices[rank]);
  if (g.err != cudaSuccess) return cuda_status(g.err);
  long long idx = 0;
  hq_shard_layout(c->world, c->rows, c->n_local, c->slots, rank, slot, nullptr, &idx, nullptr);
  unsigned char* tab = c->tables[rank];
  return hq_gather_publish(reinterpret_cast<void* const*>(tab + tl.peer_data), idx, (int)slice,
                           reinterpret_cast<uint32_t* const*>(tab + tl.peer_flags),
                           reinterpret_cast<unsigned*>(tab + tl.sync_pub), c->world, rank, 0,
                           reinterpret_cast<int*>(tab + tl.status),
                           (hq_stream_t)c->streams[rank]);
}

int hq_shard_allgather_nccl(hq_shard_ctx* c, int slot) {
  using namespace hq;
  if (!rank_ok(c, 0, slot)) return HQ_ERR_BAD_SHAPE;
  if (c->comms.empty()) return HQ_ERR_UNSUPPORTED;
  const size_t slice = (size_t)c->rows * c->n_local;
  // one grouped call over all ranks of this process, ccl-cuda/main.cu:112-117
  bool ok = c->pGroupStart() == ncclSuccess;
  for (int r = 0; ok && r < c->world; r++) {
    const void* send = hq_shard_local_slice(c, r, slot);
    void* recv = const_cast<void*>(hq_shard_gathered(c, r, slot));
    ok = c->pAllGather(send, recv, slice, ncclFloat16, c->comms[r], c->streams[r]) == ncclSuccess;
  }
  if (c->pGroupEnd() != ncclSuccess) ok = false;
  if (!ok) {
    // a failed collective leaves the communicators unusable: abort them so that
    // nothing blocks, and report
    for (auto& comm : c->comms)
      if (comm) { c->pCommAbort(comm); comm = nullptr; }
    c->comms.clear();
    return HQ_ERR_NCCL;
  }
  return HQ_OK;
}

int hq_shard_status(hq_shard_ctx* c, int rank, int* status_out) {
  using namespace hq;
  if (!rank_ok(c, rank, 0) || !status_out) return HQ_ERR_BAD_SHAPE;
  const TableLayout tl = table_layout(c->world, c->slots);
  DeviceGuard g(c->devices[rank]);
  if (g.err != cudaSuccess) return cuda_status(g.err);
  cudaError_t e = cudaStreamSynchronize(c->streams[rank]);
  if (e == cudaSuccess)
    e = cudaMemcpy(status_out, c->tables[rank] + tl.status, sizeof(int), cudaMemcpyDeviceToHost);
  return cuda_status(e);
}

}  // extern "C"
