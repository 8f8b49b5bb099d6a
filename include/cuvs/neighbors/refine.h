/* Forwarding header: keeps the include path of the reference (<cuvs/neighbors/refine.h>). */
#include "../../cuvs_refine.h"
