"""Device management (mirrors ttnn/ttnn/device.py): a device is one CUDA GPU of the local box."""
import contextlib

from . import _ttnn


def get_num_devices():
    return _ttnn.get_num_devices()


def open_device(device_id: int):
    """Open (or return the already open) device `device_id` and make it current."""
    return _ttnn.open_device(device_id)


def close_device(device):
    """Wait for outstanding work on the device. Device memory is released as its tensors go away."""
    _ttnn.close_device(device)


def synchronize_device(device):
    device.synchronize()


@contextlib.contextmanager
def manage_device(device_id: int):
    device = open_device(device_id)
    try:
        yield device
    finally:
        close_device(device)
