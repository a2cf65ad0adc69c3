// Device-memory tensor arena of the delegate.
//
// Plays the role the reference's host arena plays for delegated tensors
// (tflite/arena_planner.cc:204-382 lifetime analysis and ordering,
// tflite/simple_memory_arena.cc:370-464 greedy gap search, high-water-mark
// commit and offset -> pointer resolve): every non-constant tensor that lives
// inside a delegated partition gets an offset in ONE device slab, tensors whose
// lifetimes do not overlap share bytes, and the slab only ever grows.
// The planner itself is plain host arithmetic (no CUDA) so it is unit-tested
// on CPU; the slab is obtained through an allocator callback pair so tests can
// fake it and so the delegate's fault-injection option can fail it.
#pragma once

#include <cstddef>
#include <cstdint>
#include <vector>

namespace b200 {

struct ArenaRequest {
  size_t bytes = 0;
  int first_use = 0;  // index of the first op (in execution order) touching the tensor
  int last_use = 0;   // index of the last one; partition inputs/outputs span the whole partition
};

// Alignment of every offset. 256 B satisfies the bulk-copy (16 B) and vector
// load rules of every kernel (the reference aligns host tensors to 64 B,
// tflite/arena_planner.h:35).
constexpr size_t kArenaAlignment = 256;

// Assigns offsets; returns the slab size needed. Ordering: tensors alive for
// the whole plan first, then by size descending, ties by first use (same
// policy as ArenaPlanner::CreateTensorAllocationVector,
// tflite/arena_planner.cc:442-472); each tensor takes the smallest gap that
// fits (best fit) among the already placed tensors whose lifetimes intersect its own,
// as SimpleMemoryArena::Allocate does.
size_t PlanArena(const std::vector<ArenaRequest>& requests, int num_ops, std::vector<size_t>* offsets);

typedef void* (*ArenaAllocFn)(void* user, size_t bytes);
typedef void (*ArenaFreeFn)(void* user, void* ptr);

class DeviceArena {
 public:
  DeviceArena(ArenaAllocFn alloc, ArenaFreeFn free_fn, void* user) : alloc_(alloc), free_(free_fn), user_(user) {}
  ~DeviceArena() { Release(); }
  DeviceArena(const DeviceArena&) = delete;
  DeviceArena& operator=(const DeviceArena&) = delete;

  // Plans `requests` and makes sure the slab is large enough (re-allocating
  // only when it has to grow). False when the allocator fails.
  bool Commit(const std::vector<ArenaRequest>& requests, int num_ops);
  void* Resolve(size_t index) const {
    return index < offsets_.size() && base_ ? static_cast<uint8_t*>(base_) + offsets_[index] : nullptr;
  }
  size_t planned_bytes() const { return planned_; }
  size_t slab_bytes() const { return capacity_; }
  void Release();

 private:
  ArenaAllocFn alloc_;
  ArenaFreeFn free_;
  void* user_;
  void* base_ = nullptr;
  size_t capacity_ = 0;
  size_t planned_ = 0;
  std::vector<size_t> offsets_;
};

}  // namespace b200
