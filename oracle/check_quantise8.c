/* TEST INFRASTRUCTURE.  Exhaustive check that the 8-bit form of the layer-boundary quantiser
 * (Quantize_val, APNN-TC-nn/src/kernel.cuh:29-44: clip to [-10, 10], (v + 10) * 2^bits / 20, round to
 * nearest) can drop its division: for every float t in [0, 20] -- every value v + 10 can take after the
 * clip -- rint((t * 256) / 20) == rint(t * 12.8f), each operation rounded to float.  The GPU packers use the
 * right-hand form for 8 bits; the oracle keeps the left-hand one.  Prints the count of floats checked and
 * of mismatches, exits 0 only if there is none.
 *     gcc -O2 -mfma -ffp-contract=off -o check_quantise8 check_quantise8.c -lm && ./check_quantise8
 */
#include <stdio.h>
#include <stdint.h>
#include <string.h>
#include <math.h>
int main(){
  float hi=20.0f; uint32_t hb; memcpy(&hb,&hi,4);
  unsigned long long bad1=0,n=0;
  for(uint32_t b=0;b<=hb;b++){
    float t; memcpy(&t,&b,4);
    volatile float u=t*256.0f; volatile float q=u/20.0f; float ref=rintf(q);
    volatile float y1=t*12.8f; float c1=rintf(y1);
    if(c1!=ref){ if(bad1<5) printf("c1 t=%.9g ref=%g c1=%g\n",t,ref,c1); bad1++;}
    n++;
  }
  printf("checked=%llu mismatches=%llu\n",n,bad1);
  return bad1 ? 1 : 0;
}
