// Defined in launch.h.
#include "portdnn/matmul/launch.h"
