// The types of this header live in params.h.
#include "portdnn/conv2d/params.h"
