/* Forwarding header: keeps the include path of the reference (<cuvs/core/c_api.h>). */
#include "../../cuvs_core_c_api.h"
