// All selectors are defined in selector.h.
#include "portdnn/conv2d/selector/selector.h"
