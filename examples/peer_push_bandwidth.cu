// Peer push bandwidth between two GPUs of one machine: GPU 0 writes or add-reduces into GPU 1's memory
// with bulk copies from shared memory (the form the sharded GEMM epilogue uses), with coalesced vector
// stores and with coalesced 4-byte reductions, for several piece sizes and numbers of pushing CTAs.
// The figures size the roofline of the fused split-K exchange (aiehlc_gemm_i8_i32_scatter_dev).
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o examples/_bin/peer_push_bandwidth examples/peer_push_bandwidth.cu
//   examples/_bin/peer_push_bandwidth            (needs two GPUs with peer access; prints GB/s per case)
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("ERR %s line %d: %s\n", #x, __LINE__, cudaGetErrorString(e)); return 1; } } while (0)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// mode 0: bulk store, 1: bulk reduce add s32, 2: st.global.v4 coalesced, 3: red.global.add.s32 coalesced
__global__ void __launch_bounds__(128) push_kernel(int32_t* dst, size_t total_bytes, int piece, int mode, int row_pitch_bytes) {
  extern __shared__ __align__(128) uint8_t sm[];
  // each warp owns 2 staging buffers of `piece*rows` ... keep it simple: one piece = `piece` bytes contiguous
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = gridDim.x * 4;
  const int gw = blockIdx.x * 4 + warp;
  uint8_t* buf = sm + warp * 8192;
  for (int i = lane; i < 8192 / 4; i += 32) reinterpret_cast<int32_t*>(buf)[i] = 1;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  const size_t chunk = 4096;  // bytes per warp iteration
  const size_t n_chunks = total_bytes / chunk;
  for (size_t c = gw; c < n_chunks; c += warps) {
    uint8_t* d = reinterpret_cast<uint8_t*>(dst) + c * chunk;
    if (mode <= 1) {
      if (lane == 0) {
        for (int off = 0; off < (int)chunk; off += piece) {
          if (mode == 0)
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(d + off), "r"(smem_u32(buf + off)), "r"(piece) : "memory");
          else
            asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.s32 [%0], [%1], %2;" ::"l"(d + off), "r"(smem_u32(buf + off)), "r"(piece) : "memory");
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      }
      __syncwarp();
    } else if (mode == 2) {
      for (int off = lane * 16; off < (int)chunk; off += 512) *reinterpret_cast<int4*>(d + off) = make_int4(1, 1, 1, 1);
    } else {
      for (int off = lane * 4; off < (int)chunk; off += 128) atomicAdd(reinterpret_cast<int*>(d + off), 1);
    }
  }
  if (mode <= 1 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

int main() {
  int n = 0; CK(cudaGetDeviceCount(&n));
  if (n < 2) { printf("need 2 GPUs\n"); return 0; }
  int can = 0; CK(cudaDeviceCanAccessPeer(&can, 0, 1));
  printf("can access peer: %d\n", can);
  if (!can) return 0;
  const size_t bytes = 1ull << 30;
  int32_t *remote, *local;
  CK(cudaSetDevice(1)); CK(cudaMalloc(&remote, bytes)); CK(cudaMemset(remote, 0, bytes)); CK(cudaDeviceSynchronize());
  CK(cudaSetDevice(0)); CK(cudaDeviceEnablePeerAccess(1, 0)); CK(cudaMalloc(&local, bytes)); CK(cudaMemset(local, 0, bytes));
  CK(cudaFuncSetAttribute(push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 8192));
  cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
  const char* names[4] = {"bulk store", "bulk reduce-add", "st.v4 coalesced", "red.add.s32 coalesced"};
  for (int target = 0; target < 2; ++target) {
    int32_t* dst = target ? remote : local;
    for (int mode = 0; mode < 4; ++mode) {
      for (int piece : {128, 4096}) {
        if (mode >= 2 && piece != 128) continue;
        for (int grid : {18, 37, 74, 148, 296}) {
          push_kernel<<<grid, 128, 4 * 8192>>>(dst, bytes, piece, mode, 0);
          CK(cudaDeviceSynchronize());
          CK(cudaEventRecord(e0));
          for (int r = 0; r < 3; ++r) push_kernel<<<grid, 128, 4 * 8192>>>(dst, bytes, piece, mode, 0);
          CK(cudaEventRecord(e1)); CK(cudaDeviceSynchronize());
          float ms; CK(cudaEventElapsedTime(&ms, e0, e1));
          printf("%s %-22s piece %4d grid %3d: %7.1f GB/s\n", target ? "PEER " : "LOCAL", names[mode], piece, grid, 3.0 * bytes / ms / 1e6);
        }
      }
    }
  }
  return 0;
}
