// Defined in launch.h.
#include "portdnn/binaryop/launch.h"
