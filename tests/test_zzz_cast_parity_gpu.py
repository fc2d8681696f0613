"""Storage-type casts give the same values on the device and on the host."""
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["FP16", "BF16", "NF4", "INT8", "INT4", "FP8_E4M3", "FP8_E5M2"])
def test_casts_give_the_same_values_on_the_gpu_and_on_the_cpu(name):
    """The reference's tests/gpu_cast_test.cpp: 2 sin(i) cast to each storage type and back agrees between devices."""
    import math
    import litetorch_b200 as lt
    data = [math.sin(i) * 2.0 for i in range(128)]
    dt = getattr(lt.DataType, name)
    back = []
    for dev in (lt.Device("cpu"), lt.Device("cuda", 0)):
        t = lt.Tensor.from_vector(data, [128], dev, False)
        back.append(t.cast(dt).cast(lt.DataType.FP32).to_vector())
    assert max(abs(a - b) for a, b in zip(*back)) <= 1e-4
