// Bindings of the NVLink peer-memory collectives (comm.cu).  Peer pointers arrive as integers obtained from
// torch.distributed._symmetric_memory rendezvous handles; kernels run on the current CUDA stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

#include "kernels.h"

namespace {

using torch::Tensor;

void fill_ptrs(const std::vector<int64_t>& in, void** out, int world) {
  TORCH_CHECK((int)in.size() == world && world >= 1 && world <= seg::kMaxRanks, "need one pointer per rank (at most ", seg::kMaxRanks, ")");
  for (int i = 0; i < world; ++i) out[i] = reinterpret_cast<void*>(static_cast<uintptr_t>(in[i]));
}

void comm_allreduce_bucket(Tensor grads, std::vector<int64_t> wire_ptrs, std::vector<int64_t> flag_ptrs, int64_t mc_ptr,
                           int64_t wire_off, int64_t rank, int64_t seq, int64_t blocks, Tensor status,
                           const std::optional<Tensor>& sq_out, int64_t wait_cycles, int64_t wire_elems) {
  TORCH_CHECK(grads.is_cuda() && grads.scalar_type() == at::kFloat && grads.is_contiguous(), "grads must be a contiguous CUDA fp32 tensor");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt, "status must be a CUDA int32 tensor");
  const int world = (int)wire_ptrs.size();
  const int64_t n = grads.numel();
  TORCH_CHECK(n % (world * 8) == 0, "bucket length must be a multiple of 8 * world");
  TORCH_CHECK(wire_off % 8 == 0, "wire offset must be a multiple of 8 elements");
  TORCH_CHECK(blocks >= 1 && blocks <= seg::kCommMaxBlocks, "blocks out of range");
  void* wires[seg::kMaxRanks];
  void* flags[seg::kMaxRanks];
  fill_ptrs(wire_ptrs, wires, world);
  fill_ptrs(flag_ptrs, flags, world);
  c10::cuda::CUDAGuard guard(grads.device());
  seg::comm_allreduce_bucket(grads.data_ptr<float>(), wires, reinterpret_cast<uint32_t* const*>(flags),
                             reinterpret_cast<void*>(static_cast<uintptr_t>(mc_ptr)), wire_off, n, (int)rank, world, (uint32_t)seq,
                             (int)blocks, status.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream(),
                             sq_out.has_value() ? sq_out->data_ptr<float>() : nullptr, (long long)wait_cycles, wire_elems);
}

void comm_allgather(std::vector<int64_t> buf_ptrs, std::vector<int64_t> flag_ptrs, int64_t off_bytes, int64_t chunk_bytes,
                    int64_t rank, int64_t seq, int64_t blocks, Tensor status, int64_t wait_cycles) {
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt, "status must be a CUDA int32 tensor");
  const int world = (int)buf_ptrs.size();
  TORCH_CHECK(chunk_bytes % 16 == 0 && off_bytes % 16 == 0, "chunks must be 16-byte multiples");
  TORCH_CHECK(blocks >= 1 && blocks <= seg::kCommMaxBlocks, "blocks out of range");
  void* bufs[seg::kMaxRanks];
  void* flags[seg::kMaxRanks];
  fill_ptrs(buf_ptrs, bufs, world);
  fill_ptrs(flag_ptrs, flags, world);
  c10::cuda::CUDAGuard guard(status.device());
  seg::comm_allgather(bufs, reinterpret_cast<uint32_t* const*>(flags), off_bytes, chunk_bytes, (int)rank, world, (uint32_t)seq,
                      (int)blocks, status.data_ptr<int>(), at::cuda::getCurrentCUDAStream().stream(), (long long)wait_cycles);
}

}  // namespace

void register_comm(pybind11::module_& m) {
  m.def("comm_allreduce_bucket", &comm_allreduce_bucket, pybind11::arg("grads"), pybind11::arg("wire_ptrs"), pybind11::arg("flag_ptrs"),
        pybind11::arg("mc_ptr"), pybind11::arg("wire_off"), pybind11::arg("rank"), pybind11::arg("seq"), pybind11::arg("blocks"),
        pybind11::arg("status"), pybind11::arg("sq_out") = std::nullopt, pybind11::arg("wait_cycles") = 0,
        pybind11::arg("wire_elems") = 0);
  m.def("comm_allgather", &comm_allgather, pybind11::arg("buf_ptrs"), pybind11::arg("flag_ptrs"), pybind11::arg("off_bytes"),
        pybind11::arg("chunk_bytes"), pybind11::arg("rank"), pybind11::arg("seq"), pybind11::arg("blocks"), pybind11::arg("status"),
        pybind11::arg("wait_cycles") = 0);
  m.attr("COMM_MAX_BLOCKS") = seg::kCommMaxBlocks;
  m.attr("COMM_MAX_RANKS") = seg::kMaxRanks;
}
