/* Forwarding header: keeps the include path of the reference (<cuvs/neighbors/ivf_pq.h>). */
#include "../../cuvs_ivf_pq.h"
