/* Forwarding header: keeps the path <root>/kvx_abi.h that consumers of the KVX project
 * include (reference: kvx_abi.h).  The declarations live in include/kvx_abi.h. */
#include "include/kvx_abi.h"
