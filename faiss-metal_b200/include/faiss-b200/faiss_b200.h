// Umbrella header (include/faiss-metal/faiss_metal.h:1-7).
#pragma once
#include "B200DeviceCapabilities.h"
#include "B200Exception.h"
#include "B200IndexFlat.h"
#include "B200Resources.h"
#include "B200ShardedIndexFlat.h"
#include "StandardB200Resources.h"
