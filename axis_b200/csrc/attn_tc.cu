// tcgen05 flash attention (placeholder until the kernels land): reports
// "not served" so that the dispatcher uses the general attention kernels.
#include "kernels.h"
int ax_attn_tc_init(void) { return 0; }
int ax_attn_fwd_tc(const void*, const void*, const void*, void*, float*, const AttnShape&, int*, cudaStream_t) { return -1; }
int ax_attn_bwd_tc(const void*, const void*, const void*, const void*, const void*, const float*, float*, void*, void*, void*,
                   const AttnShape&, int*, cudaStream_t) { return -1; }
