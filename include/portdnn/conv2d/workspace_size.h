// query_workspace_size lives in launch.h.
#include "portdnn/conv2d/launch.h"
