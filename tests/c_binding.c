/* A C99 translation unit written the way a clBLAS user's would be, against include/clblas_b200.h: it must
 * compile with -std=c99 -pedantic without warnings, link against libclblas_b200.so and run without a GPU
 * (tests/test_c_binding.py).  Only calls that are decided before any device work are made. */
#include "clblas_b200.h"
#include <stdio.h>
int main(void) {
    unsigned a, b, c;
    clblasStatus st = clblasGetVersion(&a, &b, &c);
    FloatComplex z = floatComplex(1.0f, 2.0f);
    DoubleComplex w = doubleComplex(3.0, 4.0);
    printf("%d %u.%u.%u %g %g %zu %zu\n", (int)st, a, b, c, (double)CREAL(z), CIMAG(w), sizeof(FloatComplex), sizeof(DoubleComplex));
    /* NULL matrix is rejected before any device work */
    st = clblasSgemm(clblasColumnMajor, clblasNoTrans, clblasNoTrans, 4, 4, 4, 1.0f, NULL, 0, 4, NULL, 0, 4, 0.0f, NULL, 0, 4, 0, NULL, 0, NULL, NULL);
    printf("%d\n", (int)st);
    return 0;
}
