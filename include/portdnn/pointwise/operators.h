// Defined in launch.h.
#include "portdnn/pointwise/launch.h"
