/* Exhaustive check of the reciprocal-based division used by the quantizer kernel.
 *
 * q0 = RN(a*r), e = fma(-b, q0, a), q = fma(e, r, q0) with r = RN(1/b) is compared with IEEE a/b for
 * every float32 numerator mantissa and every E4M3 divisor mantissa (1, 1.125, ..., 1.875; the
 * subnormal scales k * 2^-9 have the same mantissas). Powers of two scale every step exactly, so
 * mantissas are all that matters. Prints "bad3=0" when the three-operation sequence is exact.
 * Build: gcc -O2 -mfma -ffp-contract=off exact_division_check.c -lm
 */
#include <stdio.h>
#include <math.h>
#include <stdint.h>
#include <string.h>
static float u2f(uint32_t u){float f;memcpy(&f,&u,4);return f;}
int main(){
  long bad3=0,bad5=0;
  for(int k=8;k<16;k++){
    float b=k/8.0f; float r=1.0f/b;
    for(uint32_t m=0;m<(1u<<23);m++){
      float a=u2f(0x3f800000u|m);
      float want=a/b;
      float q0=a*r; float e=fmaf(-b,q0,a); float q1=fmaf(e,r,q0);
      if(q1!=want) bad3++;
      float e1=fmaf(-b,q1,a); float q2=fmaf(e1,r,q1);
      if(q2!=want) bad5++;
    }
  }
  /* subnormal e4m3 scales k*2^-9, k=1..7: mantissas 1,1.5(3),1.25(5),1.5(6),1.75(7) covered by k/8 forms above */
  printf("bad3=%ld bad5=%ld\n",bad3,bad5);
  /* random general divisors for the 5-op sequence */
  uint64_t st=88172645463325252ull; long badg=0, badg3=0;
  for(long i=0;i<200000000;i++){
    st^=st<<13; st^=st>>7; st^=st<<17;
    float a=u2f(0x3f800000u|(uint32_t)(st&0x7fffff)); float b=u2f(0x3f800000u|(uint32_t)((st>>23)&0x7fffff));
    float r=1.0f/b; float want=a/b;
    float q0=a*r; float e=fmaf(-b,q0,a); float q1=fmaf(e,r,q0); if(q1!=want) badg3++;
    float e1=fmaf(-b,q1,a); float q2=fmaf(e1,r,q1); if(q2!=want) badg++;
  }
  printf("general: bad3=%ld bad5=%ld of 2e8\n",badg3,badg);
  return 0;
}
