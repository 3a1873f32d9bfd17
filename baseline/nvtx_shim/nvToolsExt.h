#include <nvtx3/nvToolsExt.h>
