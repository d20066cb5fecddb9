// Part of portdnn/softmax/launch.h in this implementation.
#include "portdnn/softmax/launch.h"
