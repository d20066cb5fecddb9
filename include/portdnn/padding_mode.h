// See data_format.h: all layout and padding tags live there.
#include "portdnn/data_format.h"
