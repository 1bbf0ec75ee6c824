// Which L2 partition each SM sits next to, measured: the evidence behind the design notes on the
// GPU's two L2 partitions (an operand that every SM reads is held once per partition).
//
// Atomics are carried out where their line has its home.  Every SM, one at a time (a window of the
// global timer each, so that they do not queue behind one another), times a chain of dependent
// atomics to each of 16 fixed lines about 1 MiB apart, and then a chain of dependent L1-bypassing
// loads to the same lines.  On a two-partition GPU the atomics take about 300 cycles from the SMs
// of one die and about 700 from the other, every line splitting the SMs the same way or the
// opposite way; the loads take about 300 cycles from every SM once the line has been read there,
// i.e. the far lines were copied into the near partition.
//
// Prints one line of JSON: SM count, the two group sizes (0 0 when the device shows one partition),
// mean near / far atomic latency, mean load latency near / far, and the SM-to-group map as a string.
// Every wait is on the clock and has an iteration limit; nothing here waits for another CTA.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <string>
#include <vector>

namespace {

constexpr int kLines = 16, kChain = 16, kMaxSms = 1024, kWindowNs = 60000;
constexpr size_t kStrideWords = ((size_t)1 << 18) + 264;

__device__ __forceinline__ unsigned sm_id()
{
    unsigned r;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(r));
    return r;
}
__device__ __forceinline__ unsigned long long timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void probe(unsigned* claimed, unsigned* lines, float* atom, float* load)
{
    if (threadIdx.x != 0) return;
    const unsigned sm = sm_id();
    if (sm >= (unsigned)kMaxSms || atomicAdd(&claimed[sm], 1u) != 0u) return;  // one CTA per SM measures
    const unsigned long long start = timer_ns() + (unsigned long long)sm * kWindowNs;
    for (int spin = 0; spin < (1 << 24) && timer_ns() < start; ++spin) {
    }
    for (int j = 0; j < kLines; ++j) {
        unsigned* a = lines + (size_t)j * kStrideWords;  // the lines hold zeros: the chains stay on the line
        unsigned o = atomicAdd(a, 0u);
        long long t0 = clock64();
        for (int i = 0; i < kChain; ++i) o = atomicAdd(a + (o >> 31), 0u);
        long long t1 = clock64();
        atom[sm * kLines + j] = (float)(t1 - t0) / kChain + (float)(o >> 31);
        asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(o) : "l"(a));
        t0 = clock64();
        for (int i = 0; i < kChain; ++i) {
            const unsigned* q = a + (o >> 31);
            asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(o) : "l"(q));
        }
        t1 = clock64();
        load[sm * kLines + j] = (float)(t1 - t0) / kChain + (float)(o >> 31);
    }
}

}  // namespace

int main()
{
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, 0) != cudaSuccess) return 2;
    const int sms = prop.multiProcessorCount;
    unsigned *claimed = nullptr, *lines = nullptr;
    float *atom = nullptr, *load = nullptr;
    const size_t line_bytes = (kStrideWords * kLines + 64) * sizeof(unsigned);
    cudaMalloc(&claimed, kMaxSms * sizeof(unsigned));
    cudaMalloc(&lines, line_bytes);
    cudaMalloc(&atom, (size_t)kMaxSms * kLines * sizeof(float));
    cudaMalloc(&load, (size_t)kMaxSms * kLines * sizeof(float));
    cudaMemset(claimed, 0, kMaxSms * sizeof(unsigned));
    cudaMemset(lines, 0, line_bytes);
    cudaMemset(atom, 0, (size_t)kMaxSms * kLines * sizeof(float));
    cudaMemset(load, 0, (size_t)kMaxSms * kLines * sizeof(float));
    probe<<<sms * 8, 32>>>(claimed, lines, atom, load);
    if (cudaDeviceSynchronize() != cudaSuccess) {
        std::printf("{\"error\": \"%s\"}\n", cudaGetErrorString(cudaGetLastError()));
        return 1;
    }
    std::vector<float> ha((size_t)kMaxSms * kLines), hl((size_t)kMaxSms * kLines);
    std::vector<unsigned> hc(kMaxSms);
    cudaMemcpy(ha.data(), atom, ha.size() * sizeof(float), cudaMemcpyDeviceToHost);
    cudaMemcpy(hl.data(), load, hl.size() * sizeof(float), cudaMemcpyDeviceToHost);
    cudaMemcpy(hc.data(), claimed, hc.size() * sizeof(unsigned), cudaMemcpyDeviceToHost);

    std::vector<int> seen;
    for (int s = 0; s < kMaxSms; ++s)
        if (hc[(size_t)s]) seen.push_back(s);
    bool two = (int)seen.size() * 10 >= sms * 9;  // an SM that got no CTA of the probe is left out
    std::vector<int> group(seen.size(), 0);  // 1: near to line 0
    double near_a = 0, far_a = 0, near_l = 0, far_l = 0;
    long long near_n = 0, far_n = 0;
    int lines_opposite = 0;
    for (int j = 0; j < kLines && two; ++j) {
        float lo = 1e30f, hi = 0.f;
        for (int s : seen) {
            lo = std::min(lo, ha[(size_t)s * kLines + j]);
            hi = std::max(hi, ha[(size_t)s * kLines + j]);
        }
        if (!(lo > 0.f) || hi < 1.5f * lo) {
            two = false;
            break;
        }
        const float cut = 0.5f * (lo + hi);
        size_t same = 0;
        for (size_t k = 0; k < seen.size(); ++k) {
            const bool near = ha[(size_t)seen[k] * kLines + j] < cut;
            if (j == 0) group[k] = near;
            same += (near ? 1 : 0) == group[k];
            (near ? near_a : far_a) += ha[(size_t)seen[k] * kLines + j];
            (near ? near_l : far_l) += hl[(size_t)seen[k] * kLines + j];
            ++(near ? near_n : far_n);
        }
        if (same == 0) ++lines_opposite;
        else if (same != seen.size()) two = false;  // a line that cuts the SMs differently: no clean picture
    }
    int on[2] = {0, 0};
    std::string map;
    for (size_t k = 0; k < seen.size(); ++k) {
        ++on[group[k]];
        map += group[k] ? '1' : '0';
    }
    if (!two) on[0] = on[1] = 0;
    std::printf("{\"sms\": %d, \"reporting\": %zu, \"two_partitions\": %s, \"group_sizes\": [%d, %d], \"lines\": %d, "
                "\"lines_split_the_opposite_way\": %d, \"atomic_cycles_near\": %.0f, \"atomic_cycles_far\": %.0f, "
                "\"load_cycles_near_home\": %.0f, \"load_cycles_far_home\": %.0f, \"group_of_sm\": \"%s\"}\n",
                sms, seen.size(), two ? "true" : "false", on[0], on[1], kLines, lines_opposite,
                near_n ? near_a / near_n : 0.0, far_n ? far_a / far_n : 0.0, near_n ? near_l / near_n : 0.0,
                far_n ? far_l / far_n : 0.0, two ? map.c_str() : "");
    cudaFree(claimed);
    cudaFree(lines);
    cudaFree(atom);
    cudaFree(load);
    return 0;
}
