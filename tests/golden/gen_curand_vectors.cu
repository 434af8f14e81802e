// Generates tests/golden/curand_philox_uniform.json: uniforms drawn by the CUDA toolkit's own cuRAND
// device header, compiled for the HOST (no GPU needed), for the generator arrangement the reference
// uses: curand_init(seed, subsequence, 0) followed by successive curand_uniform() calls
// (gact/gact/cpp_extension/quantization_cuda_kernel.cu:55-56,65).
//
//   nvcc -O1 -o /tmp/gen_curand gen_curand_vectors.cu && /tmp/gen_curand > curand_philox_uniform.json
#define QUALIFIERS static inline __host__ __device__
#include <curand_kernel.h>
#include <cstdio>
#include <cstdint>
#include <cstring>

int main() {
    const unsigned long long seeds[] = {0ull, 1ull, 3ull, 12345ull, 0xFFFFFFFFull, 0x100000000ull,
                                        0xDEADBEEFCAFEF00Dull};
    const unsigned long long subs[] = {0ull, 1ull, 5ull, 255ull, 256ull, 786431ull, 0xFFFFFFFFull,
                                       0x100000000ull, 0x123456789ABull};
    printf("{\"draws_per_case\": 9, \"cases\": [\n");
    bool first = true;
    for (unsigned long long seed : seeds) for (unsigned long long sub : subs) {
        curandStatePhilox4_32_10_t st;
        curand_init(seed, sub, 0ull, &st);
        printf("%s{\"seed\": %llu, \"subsequence\": %llu, \"bits\": [", first ? "" : ",\n", seed, sub);
        first = false;
        for (int i = 0; i < 9; i++) {          // 9 draws: crosses two 4-word Philox blocks
            float u = curand_uniform(&st);
            uint32_t b; memcpy(&b, &u, 4);
            printf("%s%u", i ? ", " : "", b);
        }
        printf("]}");
    }
    printf("\n]}\n");
    return 0;
}
