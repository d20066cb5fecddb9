// Part of portdnn/batchnorm/launch.h in this implementation.
#include "portdnn/batchnorm/launch.h"
