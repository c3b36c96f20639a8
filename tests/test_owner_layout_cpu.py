"""Host-only check of the weight layout of the owner-partitioned decode-step kernel: the CTAs' shares tile every matrix
exactly once, the re-packer's placement rule agrees with the order in which the kernel's consumer warps read blocks,
the streams are contiguous — for the benchmark shapes, the test architectures and odd CTA counts.  No GPU involved."""
import pytest

from seq2seqsharp_b200 import _native as N

SHAPES = {
    # name:            L,  d,    H,  Hkv, hd,  F,     V,     glu
    "c5_llama7b":     (32, 4096, 32, 8, 128, 11008, 32000, 1),
    "c3_llama1b":     (16, 2048, 32, 8, 64, 8192, 32000, 1),
    "c2_gpt2_small":  (12, 768, 12, 12, 64, 3072, 50257, 0),
    "test_gqa":       (3, 512, 8, 2, 64, 1024, 4001, 1),
    "test_hd128":     (2, 512, 4, 1, 128, 1376, 4001, 1),
    "test_mha3":      (2, 192, 3, 3, 64, 768, 4001, 0),
    "smoke":          (2, 256, 8, 2, 32, 512, 1999, 1),
    "tiny":           (1, 64, 4, 4, 16, 64, 50, 0),
}


@pytest.mark.parametrize("n_ctas", [148, 132, 37, 8])
@pytest.mark.parametrize("name", sorted(SHAPES))
def test_layout_is_consistent(native, name, n_ctas):
    L, d, H, Hkv, hd, F, V, glu = SHAPES[name]
    if Hkv > n_ctas:
        pytest.skip("fewer CTAs than KV heads: the kernel is not used")
    N.call("TSB200_OwnerLayoutSelfTest", L, d, H, Hkv, hd, F, V, glu, n_ctas)


def test_shapes_outside_the_kernel_are_refused(native):
    with pytest.raises(N.TSB200Error, match="not served"):
        N.call("TSB200_OwnerLayoutSelfTest", 2, 520, 8, 2, 65, 1024, 4001, 1, 148)     # head size not a multiple of 16
    with pytest.raises(N.TSB200Error, match="not served"):
        N.call("TSB200_OwnerLayoutSelfTest", 2, 8192, 64, 8, 128, 28672, 32000, 1, 148)  # rows wider than the staged row
