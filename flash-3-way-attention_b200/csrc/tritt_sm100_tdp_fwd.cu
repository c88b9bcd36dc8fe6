// placeholder, replaced below
#include "tritt_common.cuh"
namespace tritt {
bool sm100_tdp_supported(int, int, int, int, const TdpMask&) { return false; }
int sm100_tdp_fwd(const TdpArgs&) { set_error("not built"); return -100; }
int sm100_tdp_bwd(const TdpArgs&) { set_error("not built"); return -100; }
size_t sm100_tdp_workspace(int, int, int, int, int, int) { return 0; }
}
