// Defined in launch.h.
#include "portdnn/pooling/launch.h"
