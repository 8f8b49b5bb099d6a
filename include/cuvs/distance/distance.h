/* Forwarding header: keeps the include path of the reference (<cuvs/distance/distance.h>). */
#include "../../cuvs_distance.h"
