"""The kernel-plugin boundary (symmetrix_jit_cuda_plugin_query_v2): this library's layer-1 kernels behind the
reference's plugin interface against the reference's own generated CUDA plugin, on the same device buffers."""
import pytest

pytestmark = pytest.mark.gpu


def test_layer1_kernels_match_the_reference_generated_plugin(tmp_path):
    from oracle import kernel_ab

    report = kernel_ab.main(["--cells", "4", "--repeats", "2", "--out", str(tmp_path / "ab.json")])
    if report is None:
        pytest.skip("the reference's generated plugin (oracle/_ref) was not built")
    # the harness itself asserts the agreement of Phi1, H1_adj and the directed forces; timings are informative
    assert report["max_abs_difference"]["phi"] <= 2e-4 * max(1.0, report["max_abs_value"]["phi"])
    assert report["reference_plugin"]["forward_ms"] > 0 and report["this_library"]["reverse_ms"] > 0
