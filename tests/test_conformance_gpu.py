"""dash-conformance's attention bodies through the C ABI on the GPU, as dash-ops' own tests run
them (crates/dash-ops/tests/attention_masks.rs:326-337, :700-735): every torch record in f32, bf16
and f16, the query gradient summed both ways; a forward without gradients; decoding against
attention with one query."""
import pytest

import conformance as C
from dashmag_b200.contract import DType

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def adapter():
    from adapter import B200Adapter
    return B200Adapter()


# f32: the bound the task states is 1e-5 of the output scale; the kernels are held to the
# reference's own f32 bounds for implementations that sum in other orders (AUTOTUNE_F32, 1e-6).
@pytest.mark.parametrize("deterministic", [True, False])
@pytest.mark.parametrize("dtype,bounds", [(DType.F32, C.AUTOTUNE_F32), (DType.BF16, C.BF16), (DType.F16, C.F16)],
                         ids=["f32", "bf16", "f16"])
def test_matches_torch(adapter, dtype, bounds, deterministic):
    worst = C.matches_torch(adapter, f"b200 {dtype.name.lower()}", dtype, deterministic, bounds).all_ran()
    print("largest relative errors:", worst)


@pytest.mark.parametrize("dtype,bounds", [(DType.BF16, C.BF16), (DType.F16, C.F16)], ids=["bf16", "f16"])
def test_matches_torch_on_the_tensor_core_kernels(adapter, dtype, bounds):
    """The same ten records with the size rule lifted (dash_attn_force_tensor), so that the tcgen05
    kernels themselves meet the reference's recorded vectors, as the reference's fast kernels do:
    the D = 64 records through the two-tile forward and both backward kernels, the D = 256 record
    through the one-tile forward and the half-tile passes of the backward.  The bounds
    are dash-conformance's own (crates/dash-conformance/src/attention.rs:99-108)."""
    from dashmag_b200 import _lib
    lib = _lib.lib()
    before = _lib.probe("tensor_core_runs")
    lib.dash_attn_force_tensor(1)
    try:
        worst = C.matches_torch(adapter, f"b200 tcgen05 {dtype.name.lower()}", dtype, True, bounds).all_ran()
    finally:
        lib.dash_attn_force_tensor(0)
    ran = _lib.probe("tensor_core_runs") - before
    assert ran == 20, f"only {ran} of the records' 20 passes ran on the tensor cores"
    print("largest relative errors on the tensor-core kernels:", worst)


def test_forward_without_gradients(adapter):
    C.without_gradients(adapter, "b200", C.AUTOTUNE_F32).all_ran()


def test_decoding_is_attention_with_one_query(adapter):
    # Absolute bounds; the decoding kernel and the training kernel sum in different orders, so the
    # reference's "to the bit" (its CPU path decodes through the same code) becomes f32 rounding.
    C.decoding_is_attention_with_one_query(adapter, "b200", [1e-6, 1e-6]).all_ran()
