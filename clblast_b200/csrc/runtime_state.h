// Per-process state shared by the C-ABI layer and the kernel launchers: the SM count of each device, the key that
// identifies the current context, and the status block through which the tensor-core kernels report an expired
// bounded wait.
#pragma once

#include <cuda_runtime_api.h>

#include <atomic>

namespace b200 {

// Number of SMs of the current device (queried once per device ordinal; safe to call from any thread).
int sm_count();

// table[current device], computed with `compute` on first use (e.g. the number of resident CTA pairs of a kernel).
// Values <= 0 are returned but not cached; -1 when the device ordinal does not fit the table.
constexpr int kMaxDevices = 64;
int per_device(std::atomic<int> (&table)[kMaxDevices], int (*compute)());

// Key of the context current on the calling thread: the driver's unique context id where available (a destroyed
// context's handle value can be reused), else the handle value. Binds the primary context when none is current.
// Returns 0 and stores the key, or a CUresult / cudaError value.
int context_key(unsigned long long* key);

// Raises a kernel's dynamic shared-memory limit to `smem_bytes` unless this context already has it at least that high,
// and returns the kernel's register count in `regs` when asked. The runtime calls behind this take a few microseconds
// per launch otherwise, which is what a small problem's kernel takes. `func` is the kernel's host function pointer.
cudaError_t kernel_ready(const void* func, int smem_bytes, int* regs = nullptr);

// Status block written by the tensor-core kernels when a bounded wait expires: word 0 = code (1 producer,
// 2 accumulator-free, 3 operands-ready, 4 accumulator-ready, 5 raw-tile, 6 old-C block), word 1 = block index,
// word 2 = barrier address. It lives in a page of host memory inside the library image that is registered with the
// driver as mapped, portable pinned memory, so kernels of every context write it directly and the host reads it
// without a copy or a stream operation (after synchronising the stream the kernel ran on). Nothing is allocated.
// Returns the device-visible address, or null when the registration failed (kernels then skip the report).
unsigned int* tc_status_device();

// Copies the status block to `out` and, with `clear`, resets a non-zero block. Meaningful after the stream that ran
// the kernel has been synchronised. Returns false when the block is unavailable.
bool tc_status_read(unsigned int out[4], bool clear);

}  // namespace b200
