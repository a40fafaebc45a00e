/*
 * The reference's own transfer path, restated for timing beside the product.
 *
 * TEST / BENCHMARK INFRASTRUCTURE ONLY — never linked into the product library.
 *
 * What a reference GPU worker does for one task (pegaflow-core/src/gpu_worker.rs:428-523):
 *   1. build one CopyDesc per (layer, block, segment)        gpu_worker.rs:353-423
 *   2. hand the batch to the backend
 *        direct: coalesce neighbours, one cuMemcpy{HtoD,DtoH}Async per range   transfer/memcpy.rs:25-97
 *        kernel: flatten to [dst,src,size] u64 triples, pageable upload into a grow-only
 *                device buffer, one launch of clamp(n,1,65535) x 256 threads   transfer/kernel.rs:79-135
 *   3. record an event and wait for it                        gpu_worker.rs:444-449,497-502
 * Steps 1 and the coalescing of step 2 come from the C oracle (pf_oracle.c); this file adds
 * the CUDA calls.  The reference's kernel itself is not restated: when the reference checkout
 * is present at build time its CUDA source string is extracted, compiled here unchanged
 * (PF_REF_KERNEL_INC) and only the binary is kept.
 */
#include <cuda_runtime.h>

#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "pf_oracle.h"

#ifdef PF_REF_KERNEL_INC
#include PF_REF_KERNEL_INC
#endif

static double now_s(void) {
  struct timespec t;
  clock_gettime(CLOCK_MONOTONIC, &t);
  return (double)t.tv_sec + 1e-9 * (double)t.tv_nsec;
}

extern "C" {

typedef struct pfr_layer {
  pfo_layout layout;
  uint64_t host_base[2];     /* host address of block 0's segment s */
  uint64_t host_dev_base[2]; /* device-visible address of the same */
  size_t host_stride;        /* bytes between consecutive blocks' images */
  size_t allocation[2];
} pfr_layer;

/* Host-side bookkeeping of one task: the per-block host images a save/load carries
 * (offload.rs:477-508 / lib.rs:857-873) and the descriptor batch built from them.
 * Returns a malloc'd descriptor array; *seconds is the CPU time spent. */
pfo_copy_desc *pfr_build(const pfr_layer *layers, size_t n_layers, const size_t *block_ids, size_t n_blocks,
                         size_t *n_descs, double *seconds) {
  double t0 = now_s();
  pfo_layer_task *tasks = (pfo_layer_task *)calloc(n_layers ? n_layers : 1, sizeof(pfo_layer_task));
  size_t cap = 0;
  for (size_t li = 0; li < n_layers; ++li) {
    const pfr_layer *L = &layers[li];
    pfo_host_block *hb = (pfo_host_block *)calloc(n_blocks ? n_blocks : 1, sizeof(pfo_host_block));
    const size_t nseg = L->layout.split ? 2 : 1;
    for (size_t b = 0; b < n_blocks; ++b) {
      hb[b].block_idx = block_ids[b];
      hb[b].n_segments = nseg;
      for (size_t s = 0; s < nseg; ++s) {
        hb[b].seg_host[s] = L->host_base[s] + b * L->host_stride;
        hb[b].seg_host_device[s] = L->host_dev_base[s] + b * L->host_stride;
        hb[b].seg_allocation[s] = L->allocation[s];
      }
    }
    tasks[li].layout = L->layout;
    tasks[li].n_blocks = n_blocks;
    tasks[li].blocks = hb;
    cap += 2 * n_blocks;
  }
  pfo_copy_desc *out = (pfo_copy_desc *)malloc((cap ? cap : 1) * sizeof(pfo_copy_desc));
  char err[256];
  long n = pfo_build_copy_descs(tasks, n_layers, out, cap, NULL, err, sizeof err);
  for (size_t li = 0; li < n_layers; ++li) free((void *)tasks[li].blocks);
  free(tasks);
  if (n < 0) {
    free(out);
    out = NULL;
    n = 0;
  }
  *n_descs = (size_t)n;
  if (seconds) *seconds = now_s() - t0;
  return out;
}

void pfr_free(void *p) { free(p); }

/* transfer/memcpy.rs:61-97: one async copy per coalesced range; no synchronisation. */
int pfr_submit_direct(const pfo_copy_desc *descs, size_t n, int host_is_src, void *stream, size_t *n_calls) {
  pfo_copy_desc *merged = (pfo_copy_desc *)malloc((n ? n : 1) * sizeof(pfo_copy_desc));
  size_t m = pfo_merge(descs, n, merged);
  cudaError_t e = cudaSuccess;
  for (size_t i = 0; i < m && e == cudaSuccess; ++i) {
    if (host_is_src)
      e = cudaMemcpyAsync((void *)(uintptr_t)merged[i].device, (const void *)(uintptr_t)merged[i].host, merged[i].size,
                          cudaMemcpyHostToDevice, (cudaStream_t)stream);
    else
      e = cudaMemcpyAsync((void *)(uintptr_t)merged[i].host, (const void *)(uintptr_t)merged[i].device, merged[i].size,
                          cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  }
  free(merged);
  if (n_calls) *n_calls = m;
  return (int)e;
}

int pfr_has_reference_kernel(void) {
#ifdef PF_REF_KERNEL_INC
  return 1;
#else
  return 0;
#endif
}

static unsigned long long *g_scratch = NULL;
static size_t g_scratch_len = 0;

/* transfer/kernel.rs:79-135 with the reference's own kernel. */
int pfr_submit_kernel(const pfo_copy_desc *descs, size_t n, int host_is_src, void *stream) {
#ifdef PF_REF_KERNEL_INC
  if (n == 0) return 0;
  unsigned long long *flat = (unsigned long long *)malloc(n * 3 * sizeof(unsigned long long));
  for (size_t i = 0; i < n; ++i) {
    flat[3 * i + 0] = host_is_src ? descs[i].device : descs[i].host_device;
    flat[3 * i + 1] = host_is_src ? descs[i].host_device : descs[i].device;
    flat[3 * i + 2] = descs[i].size;
  }
  cudaError_t e = cudaSuccess;
  if (g_scratch_len < n * 3) {
    if (g_scratch) cudaFree(g_scratch);
    e = cudaMalloc(&g_scratch, n * 3 * sizeof(unsigned long long));
    g_scratch_len = e == cudaSuccess ? n * 3 : 0;
  }
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(g_scratch, flat, n * 3 * sizeof(unsigned long long), cudaMemcpyHostToDevice,
                        (cudaStream_t)stream); /* pageable source: consumed before the call returns */
  free(flat);
  if (e != cudaSuccess) return (int)e;
  unsigned grid = n > 65535 ? 65535u : (unsigned)n;
  pega_batch_copy<<<grid, 256, 0, (cudaStream_t)stream>>>(g_scratch, (int)n);
  return (int)cudaGetLastError();
#else
  (void)descs; (void)n; (void)host_is_src; (void)stream;
  return -1;
#endif
}

/* pinned_mem.rs:153-163 `allocate_cuda_host_alloc`: the pool's default backing, one
 * cudaHostAlloc(Mapped) region and its device-visible address.  The reference arm of the
 * benchmark carves its host images out of this region with a bump pointer, so that it does not
 * depend on the product library for anything. */
int pfr_host_alloc(size_t bytes, void **host, uint64_t *host_device) {
  void *p = NULL, *d = NULL;
  cudaError_t e = cudaHostAlloc(&p, bytes, cudaHostAllocMapped);
  if (e != cudaSuccess) return (int)e;
  e = cudaHostGetDevicePointer(&d, p, 0);
  if (e != cudaSuccess) {
    cudaFreeHost(p);
    return (int)e;
  }
  *host = p;
  *host_device = (uint64_t)(uintptr_t)d;
  return 0;
}

int pfr_host_free(void *host) { return (int)cudaFreeHost(host); }

/* gpu_worker.rs:444-449: record an event on the stream and wait for it. */
int pfr_sync(void *stream) {
  cudaEvent_t ev;
  cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
  if (e != cudaSuccess) return (int)e;
  e = cudaEventRecord(ev, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaEventSynchronize(ev);
  cudaEventDestroy(ev);
  return (int)e;
}

}  /* extern "C" */
