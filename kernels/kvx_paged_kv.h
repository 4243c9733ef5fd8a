/* Forwarding header: keeps the path <root>/kernels/kvx_paged_kv.h (reference:
 * kernels/kvx_paged_kv.h).  The declarations live in include/kvx_paged_kv.h. */
#include "../include/kvx_paged_kv.h"
