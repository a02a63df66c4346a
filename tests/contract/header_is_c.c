/* The public headers must also compile as plain C. */
#include "shaobo_fa3_api.h"
#include "shaobo_fa3_components.h"
int main(void) { return sizeof(ShaoboFa3Params) == 296 ? 0 : 1; }
