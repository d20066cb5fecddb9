// Defined in launch.h.
#include "portdnn/depthwise_conv2d/launch.h"
