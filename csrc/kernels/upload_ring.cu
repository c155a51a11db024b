// Pinned upload ring: a host-to-device write is cut into chunks, each staged through one slot of a small ring of
// pinned host buffers, so the host fills slot k + 1 (a read of the memory-mapped checkpoint: page faults, disk) while
// the copy engine drains slot k.  Four slots of up to 64 MiB, asynchronous copies, one event per slot - the policy of
// the reference's ring (crates/poot-runtime-common/src/ring.rs:1-17).  Host code only; it lives in this library because
// this is the one linked against the CUDA runtime.  One cudaMemcpyAsync per chunk (no batched copy calls).
#include "common.cuh"
#include <cstring>
#include <new>

namespace {

constexpr int kSlots = 4;
constexpr size_t kChunk = (size_t)64 << 20;
constexpr size_t kMinSlot = (size_t)64 << 10;

struct Ring {
  void* slot[kSlots];
  cudaEvent_t done[kSlots];
  bool in_flight[kSlots];
  size_t slot_bytes;
  int next;
  unsigned long long bytes, chunks, waits;
};

size_t slot_size(size_t need) {
  size_t p = kMinSlot;
  while (p < need && p < kChunk) p <<= 1;
  return p;
}

}  // namespace

// slot_hint: the largest write expected (a slot is the next power of two, at least 64 KiB, at most 64 MiB).
POOT_API int poot_ring_create(unsigned long long slot_hint, void** out) {
  Ring* r = new (std::nothrow) Ring();
  if (r == nullptr) return (int)cudaErrorMemoryAllocation;
  r->slot_bytes = slot_size((size_t)slot_hint);
  r->next = 0;
  r->bytes = r->chunks = r->waits = 0;
  for (int i = 0; i < kSlots; ++i) { r->slot[i] = nullptr; r->done[i] = nullptr; r->in_flight[i] = false; }
  for (int i = 0; i < kSlots; ++i) {
    cudaError_t e = cudaHostAlloc(&r->slot[i], r->slot_bytes, cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&r->done[i], cudaEventDisableTiming);
    if (e != cudaSuccess) {
      for (int j = 0; j <= i; ++j) {
        if (r->done[j]) cudaEventDestroy(r->done[j]);
        if (r->slot[j]) cudaFreeHost(r->slot[j]);
      }
      delete r;
      return (int)e;
    }
  }
  *out = r;
  return 0;
}

// Copy nbytes from pageable host memory `src` to device memory `dst` on `stream`.  Returns once every chunk is
// enqueued; the last chunks may still be in flight (poot_ring_drain waits for them).  The cursor moves only after a
// slot was ready, so a failed wait leaves it where it was.
POOT_API int poot_ring_upload(void* ring, const void* src, unsigned long long nbytes, void* dst, cudaStream_t stream) {
  Ring* r = static_cast<Ring*>(ring);
  if (r == nullptr || (nbytes != 0 && (src == nullptr || dst == nullptr))) return (int)cudaErrorInvalidValue;
  const char* s = static_cast<const char*>(src);
  char* d = static_cast<char*>(dst);
  for (unsigned long long off = 0; off < nbytes; off += r->slot_bytes) {
    const size_t n = (size_t)((nbytes - off < r->slot_bytes) ? nbytes - off : r->slot_bytes);
    const int k = r->next;
    if (r->in_flight[k]) {
      if (cudaEventQuery(r->done[k]) == cudaErrorNotReady) ++r->waits;
      cudaError_t e = cudaEventSynchronize(r->done[k]);
      if (e != cudaSuccess) return (int)e;
      r->in_flight[k] = false;
    }
    std::memcpy(r->slot[k], s + off, n);
    cudaError_t e = cudaMemcpyAsync(d + off, r->slot[k], n, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaEventRecord(r->done[k], stream);
    if (e != cudaSuccess) return (int)e;
    r->in_flight[k] = true;
    r->next = (k + 1) % kSlots;
    r->bytes += n;
    ++r->chunks;
  }
  return 0;
}

POOT_API int poot_ring_drain(void* ring) {
  Ring* r = static_cast<Ring*>(ring);
  if (r == nullptr) return (int)cudaErrorInvalidValue;
  for (int i = 0; i < kSlots; ++i)
    if (r->in_flight[i]) {
      cudaError_t e = cudaEventSynchronize(r->done[i]);
      if (e != cudaSuccess) return (int)e;
      r->in_flight[i] = false;
    }
  return 0;
}

// out4 = {bytes uploaded, chunks, waits for a busy slot, bytes of one slot}
POOT_API int poot_ring_stats(void* ring, unsigned long long* out4) {
  Ring* r = static_cast<Ring*>(ring);
  if (r == nullptr) return (int)cudaErrorInvalidValue;
  out4[0] = r->bytes; out4[1] = r->chunks; out4[2] = r->waits; out4[3] = r->slot_bytes;
  return 0;
}

POOT_API int poot_ring_destroy(void* ring) {
  Ring* r = static_cast<Ring*>(ring);
  if (r == nullptr) return 0;
  int rc = poot_ring_drain(ring);
  for (int i = 0; i < kSlots; ++i) {
    if (r->done[i]) cudaEventDestroy(r->done[i]);
    if (r->slot[i]) cudaFreeHost(r->slot[i]);
  }
  delete r;
  return rc;
}

// The policy as pure functions, for checks without a device: slot size for a hint, and the number of chunks of a write.
POOT_API unsigned long long poot_ring_slot_bytes(unsigned long long need) { return slot_size((size_t)need); }
POOT_API unsigned long long poot_ring_chunk_count(unsigned long long nbytes, unsigned long long slot_bytes) {
  return slot_bytes == 0 ? 0 : (nbytes + slot_bytes - 1) / slot_bytes;
}
