"""tt_lib.device: CreateDevice / CloseDevice / Synchronize (tt_eager/tt_lib/csrc/tt_lib_bindings.cpp)."""
import ttnn


def CreateDevice(device_id: int = 0):
    return ttnn.open_device(device_id)


def CloseDevice(device):
    ttnn.close_device(device)


def Synchronize(device=None):
    if device is not None:
        ttnn.synchronize_device(device)


def GetNumAvailableDevices():
    return ttnn._ttnn.get_num_devices()
