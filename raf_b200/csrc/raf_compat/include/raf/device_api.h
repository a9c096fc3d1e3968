// raf_compat: nothing of include/raf/device_api.h is needed by the b200 dialect beyond the
// Device type, which raf/value.h defines.
#pragma once
#include "raf/value.h"
