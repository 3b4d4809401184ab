"""Safetensors weights into an instance: poly_b200_instance_import_weights against
polygrad's own poly_instance_export_weights / poly_instance_import_weights
(src/instance.c:505-550).  Bit-exact: float32 tensors are copied, bfloat16 and
float16 tensors are widened exactly.

The CPU cases run the product library in its dry-run mode (device memory is
host memory there, copies are real, launches are ignored), in a child process
because the mode is read once at initialisation; the GPU case moves real
device buffers and checks the forward result against the CPU reference."""
import json
import os
import struct
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def safetensors_blob(tensors):
    """{name: (dtype string, shape, raw bytes)} -> safetensors bytes (8-byte little-endian header length,
    JSON header, data)."""
    header, data = {}, b''
    for name, (dtype, shape, raw) in tensors.items():
        header[name] = dict(dtype=dtype, shape=list(shape), data_offsets=[len(data), len(data) + len(raw)])
        data += raw
    h = json.dumps(header, separators=(',', ':')).encode()
    return struct.pack('<Q', len(h)) + h + data


def to_bf16_bits(a):
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


CHILD = '''
import sys
sys.path.insert(0, %(root)r)
sys.path.insert(0, %(root)r + '/tests')
import numpy as np
from polygrad_b200 import ffi
from polygrad_b200.instance import Instance
from test_weights import safetensors_blob, to_bf16_bits
lib = ffi.product()
src = Instance.mlp(lib, [20, 16, 4], 'relu', True, 2, seed=1)
rng = np.random.default_rng(3)
want = {n: rng.standard_normal(src.shape(n)).astype(np.float32) for n in src.params}
for n, a in want.items():
    src.write(n, a)
blob = src.export_weights()                       # polygrad's own encoder, float32

dst = Instance.mlp(lib, [20, 16, 4], 'relu', True, 2, seed=2)
dst.set_device(ffi.DEVICE_CUDA)
moved = dst.import_weights(blob)
assert moved == sum(a.nbytes for a in want.values()), moved
for n, a in want.items():
    assert np.array_equal(dst.read(n), a), n

# the reference call on the same instance leaves the device buffers as they were
dst2 = Instance.mlp(lib, [20, 16, 4], 'relu', True, 2, seed=2)
before = {n: dst2.read(n).copy() for n in dst2.params}
dst2.set_device(ffi.DEVICE_CUDA)
assert lib.poly_instance_import_weights(dst2.h, blob, len(blob)) == 0
assert all(np.array_equal(dst2.read(n), before[n]) for n in before)

# 16-bit files: widened exactly
b16 = {n: ('BF16', a.shape, to_bf16_bits(a).tobytes()) for n, a in want.items()}
dst.import_weights(safetensors_blob(b16))
for n, a in want.items():
    exp = (to_bf16_bits(a).astype(np.uint32) << 16).view(np.float32).reshape(a.shape)
    assert np.array_equal(dst.read(n), exp), n
f16 = {n: ('F16', a.shape, a.astype(np.float16).tobytes()) for n, a in want.items()}
dst.import_weights(safetensors_blob(f16))
for n, a in want.items():
    assert np.array_equal(dst.read(n), a.astype(np.float16).astype(np.float32)), n

# host-resident instance: filled in place, nothing goes to a device
host = Instance.mlp(lib, [20, 16, 4], 'relu', True, 2, seed=2)
assert host.import_weights(blob) == 0
for n, a in want.items():
    assert np.array_equal(host.read(n), a), n

# errors: a size mismatch and an integer tensor are refused, an unknown name is skipped
name = src.params[0]
for bad in (safetensors_blob({name: ('F32', (3,), np.zeros(3, np.float32).tobytes())}),
            safetensors_blob({name: ('I32', want[name].shape, np.zeros(want[name].size, np.int32).tobytes())}),
            b'not a safetensors file'):
    try:
        dst.import_weights(bad)
    except RuntimeError:
        pass
    else:
        raise AssertionError('accepted a bad file')
assert dst.import_weights(safetensors_blob({'no.such.tensor': ('F32', (1,), np.zeros(1, np.float32).tobytes())})) == 0
print('ok')
'''


def test_import_weights_in_dry_run():
    env = dict(os.environ, POLY_B200_DRYRUN='1', POLY_B200_DRYRUN_NOCOMPILE='1')
    r = subprocess.run([sys.executable, '-c', CHILD % dict(root=ROOT)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.strip().endswith('ok'), r.stderr[-4000:]


@pytest.mark.gpu
def test_imported_weights_drive_the_forward(ref_lib, gpu):
    """Export from a CPU instance, import into a device-resident one with other parameters, run the
    forward: the MLP output matches the CPU reference within 1e-5 and the parameters read back bit-exact."""
    from conftest import assert_close
    from polygrad_b200 import ffi
    from polygrad_b200.instance import Instance
    layers = [784, 512, 10]
    rng = np.random.default_rng(21)
    x = rng.standard_normal((256, 784)).astype(np.float32)
    cpu = Instance.mlp(ref_lib, layers, 'relu', True, 256, seed=5)
    cpu.forward(x=x)
    want = cpu.read('output')
    blob = cpu.export_weights()
    dev = Instance.mlp(gpu, layers, 'relu', True, 256, seed=99)
    dev.set_device(ffi.DEVICE_CUDA)
    moved = dev.import_weights(blob)
    assert moved == 4 * (784 * 512 + 512 + 512 * 10 + 10)
    for n in cpu.params:
        assert np.array_equal(dev.read(n), cpu.read(n)), n
    dev.forward(x=x)
    assert_close(dev.read('output'), want, 1e-5, 'mlp output after import')
    cpu.free()
    dev.free()
