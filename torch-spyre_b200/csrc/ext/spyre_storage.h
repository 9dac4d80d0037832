// Storage of a `spyre` tensor: CUDA device memory holding a stick image.
//
// The reference keeps a flex device allocation behind at::DataPtr with a
// SharedOwnerCtx context (torch_spyre/csrc/spyre_mem.cpp:486-554, module.h:27-30).
// Here the allocation comes from PyTorch's CUDA caching allocator (device memory
// and streams are PyTorch's job; `spyre:N` is CUDA device N) and the context
// additionally records the logical shape the allocation was laid out for: the
// storage is the generic stick image (SpyreTensorLayout) of a row-major tensor of
// that "base shape".  A tensor's sizes / strides / storage offset address elements
// of that row-major base, exactly as they would on the host.
#pragma once

#include <ATen/ATen.h>
#include <c10/core/Allocator.h>

#include <cstdint>
#include <vector>

namespace spyre {

constexpr int64_t kBytesInStick = 128;  // torch_spyre/csrc/spyre_tensor_impl.cpp:27

struct StorageCtx {
  void* ptr = nullptr;
  size_t nbytes = 0;
  c10::DeviceIndex device = 0;
  int elem_bytes = 0;               // 0 until a tensor has been laid out in it
  std::vector<int64_t> base_shape;  // row-major logical shape of the image
};

// Whole-stick byte size of the image of a tensor of this shape
// (torch_spyre/csrc/spyre_mem.cpp:598-611; a 0-dim tensor is laid out as [1]).
int64_t stick_nbytes(c10::IntArrayRef shape, int64_t elem_bytes);

at::Allocator* spyre_allocator();

// Context of a spyre tensor's storage (throws if the tensor is not on spyre).
StorageCtx* storage_ctx(const at::Tensor& t);

// True when the tensor covers its whole storage in row-major order with the same
// innermost extent as the base shape, i.e. the storage *is* the tensor's own generic
// stick image.
bool is_canonical(const at::Tensor& t);

// CUDA uint8 tensor aliasing the storage bytes (keeps the storage alive).
at::Tensor storage_as_cuda_bytes(const at::Tensor& t);

// Device-to-device copies of views go image to image in one pass (ts_transpose_tiles) when this
// is on (the default); off sends them through a row-major temporary, which tests compare against.
bool restickify_enabled();
void set_restickify_enabled(bool on);

void register_debug_flag();
bool debug_enabled();

}  // namespace spyre
