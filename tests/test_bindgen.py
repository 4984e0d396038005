"""The binding generator on small sources written for this test (no GPU): which kernels it recognises, what it
emits, and what it leaves of the host part."""
from aiehlc_b200 import bindgen

ABSOLUTE_WINDOWS = """
#define LEN 64
#define N 8
///* a line comment that contains a block-comment opener
__global__ void tile_mm(input_window_int32 * win __attribute__((annotate("mem_address:0x2000"), annotate("size_hint:128"))),
        output_window_int32 *res __attribute__((annotate("mem_address:0x4000")))) {
#define DEPTH 8
    uint32_t * p_out = (uint32_t *)(0x70000 + 0x4800);
    uint32_t * p_in = (uint32_t *)(0x70000 + 0x2800);
    uint32_t * a = p_in, * b = p_in + LEN;
    for (int i = 0; i < N; i++)
        for (int j = 0; j < N; j++) {
            uint32_t s = 0;
            for (int k = 0; k < N; k++) s += a[i * N + k] * b[j * N + k];
            p_out[i * N + j] = s;
        }
}
int host_code_uses(void) { return DEPTH + LEN; }   /* after the kernel */
"""

WINDOW_API = """
#define N 4
__global__ void vec_mm(input_window_int32 * win, output_window_int32 *out) {
    int32_t A[16], B[16], R[16];
    for (unsigned w = 0; w < 2; w++) chess_prepare_for_pipelining {
        aie::vector<int32_t, 16> t = window_readincr_v<16>(win);
    }
    for (int i = 0; i < N; i++) for (int j = 0; j < N; j++) for (int k = 0; k < N; k++)
        R[i*N + j] += A[i*N + k] * B[j*N + k];
    window_writeincr(out, aie::load_v<16>(R));
}
"""

PLAIN_AND_ENDLESS = """
#define CORE_IP_MEM 0x1000
#define CORE_OP_MEM 0x5000
__global__ void add_seven(int *in, int *out) {
    for (int i = 0; i < 12; ++i) out[i] = in[0] + 7;   // uses "while (1)" only in this comment
}
__global__ void spin(int *in, int *out) { while (1) { *out = *in; } }
__global__ void vector_only(input_window_int32 *w, output_window_int32 *out) {
    aie::vector<int32_t, 8> v = window_readincr_v<8>(w);
}
"""


def test_matmul_over_fixed_tile_addresses():
    (k,) = bindgen.parse_kernels(ABSOLUTE_WINDOWS)
    assert (k.name, k.kind, k.n) == ("tile_mm", "matmul", 8)
    assert (k.in_addr, k.out_addr) == (0x2800, 0x4800)         # the addresses the body uses win over the annotations
    text, _ = bindgen.generate(ABSOLUTE_WINDOWS, "a test source")
    assert "XAie_KernelBind((const void*)tile_mm" in text and "{8, 8, 8}" in text and "0x2800, 0x4800" in text
    assert "_cuda" not in text                                  # the body itself is never compiled for the GPU


def test_matmul_written_in_the_window_api_is_the_same_kernel():
    (k,) = bindgen.parse_kernels(WINDOW_API)
    assert (k.kind, k.n, k.in_addr, k.out_addr) == ("matmul", 4, 0x1000, 0x6000)


def test_plain_kernels_are_re_emitted_and_the_rest_is_reported():
    text, kernels = bindgen.generate(PLAIN_AND_ENDLESS)
    kinds = {k.name: k.kind for k in kernels}
    assert kinds == {"add_seven": "plain", "spin": "unsupported", "vector_only": "unsupported"}
    plain = kernels[0]
    assert (plain.in_addr, plain.out_addr) == (0x1000, 0x5000)  # the file's CORE_IP_MEM / CORE_OP_MEM
    assert "__global__ void add_seven_cuda(int * in, int * out)" in text and "out[i] = in[0] + 7;" in text
    assert "add_seven_cuda<<<1, 1, 0, (cudaStream_t)info->stream>>>((int *)(info->in), (int *)(info->out));" in text
    assert "spin: not bound (does not terminate)" in text and "vector_only: not bound" in text
    assert "spin_cuda" not in text


def test_host_part_keeps_the_macros_and_loses_the_kernel():
    host = bindgen.host_source(ABSOLUTE_WINDOWS)
    assert "#define DEPTH 8" in host and "int host_code_uses(void)" in host
    assert "0x70000" not in host and "s += a[" not in host
    assert host.count("__global__ void tile_mm") == 1           # the declaration stays: its address names the kernel
    host2 = bindgen.host_source(WINDOW_API)
    assert "aie::" not in host2 and "chess_" not in host2
