/* Forwarding translation unit: keeps the source path <root>/kernels/kvx_paged_kv.cu that the
 * reference's vLLM patch adds to the extension's source list (patches/vllm/kvx.patch:25-32).
 * The launch layer and kernels live in kvx_b200/csrc/kvx_paged_kv.cu, a single
 * self-contained translation unit. */
#include "../kvx_b200/csrc/kvx_paged_kv.cu"
