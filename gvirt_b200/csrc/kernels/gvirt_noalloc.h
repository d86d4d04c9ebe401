// Allocation-free entry point for paged decode attention.
//
// This entry point has no counterpart in the reference runtime; it exists for callers of this
// library that are not allowed to allocate device memory themselves and cannot hand the kernel
// a scratch buffer: plug-ins running inside another framework's memory pool whose allocator they
// must not re-enter, code running in a region where allocation is forbidden (for example while a
// stream is being captured, or in a real-time serving loop with a fixed memory budget), and C
// callers without a CUDA allocator of their own.
//
// gv_paged_attention_decode needs scratch for split-KV (partial outputs + log-sum-exps) and takes
// it as two pointers. This variant keeps that scratch in a fixed array that lives inside the
// library image (GV_NOALLOC_SCRATCH_BYTES on every GPU that loads the library, held until the
// process exits), so the caller passes only inputs and the output.
//
// Contract:
//   * Required scratch = batch * nq * nsplit * (head_dim + 1) * 4 bytes. A call that needs more
//     than GV_NOALLOC_SCRATCH_BYTES is rejected with GV_ETOOBIG (-4) and a message in
//     gv_last_error(); nothing is launched. nsplit == 1 needs no scratch at all.
//   * The first call on each device resolves the device address of the array (and of a private
//     status word) with cudaGetSymbolAddress. That set-up is a host-side query; make that first
//     call during start-up, before beginning any stream capture on that device.
//   * No cudaMalloc / cudaFree / allocating library routine is called, on any call.
//   * All calls on a device share the one array and it keeps the previous call's contents. The
//     kernel fully overwrites every partial slot it later reads, so nothing has to be cleared
//     between calls — but two calls whose kernels overlap on the GPU (different streams without
//     an ordering between them) race on the array. Serialise them on one stream or with events.
//   * Arguments and results are otherwise identical to gv_paged_attention_decode. The raw
//     metadata is not validated on the host: a sequence length beyond max_blocks * block_size or
//     a block id outside [0, num_blocks) raises GV_ST_BAD_INDEX (32) in the status word below
//     and the affected keys are skipped; nothing is read out of range.
//   * The entry points may be called from several host threads; the per-device set-up is
//     serialised internally.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

#define GV_NOALLOC_SCRATCH_BYTES (8u << 20)

int gv_paged_attention_decode_noalloc(const void* q, const void* k_cache, const void* v_cache,
                                      const void* block_tables, const void* seq_lens, void* out,
                                      long long batch, long long nq, long long nkv,
                                      long long head_dim, long long block_size,
                                      long long max_blocks, long long nsplit, float scale,
                                      long long num_blocks, void* stream);

// Bits raised by kernels launched through the entry point above on the current device
// (same meaning as the library-wide status word); synchronises `stream`.
int gv_noalloc_status_read(unsigned int* host_out, void* stream);
// Clears those bits (an asynchronous memset on `stream`): the word is sticky, so a caller that has
// handled an error clears it before the next call it wants to check.
int gv_noalloc_status_reset(void* stream);

#ifdef __cplusplus
}
#endif
