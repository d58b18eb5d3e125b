"""Kernel registry, mirroring tfjs-core/src/kernel_registry.ts.

A kernel is registered under `${backendName}_${kernelName}` (kernel_registry.ts:
206-209) with the names of tfjs-core/src/kernel_names.ts; `kernelFunc` receives
{inputs, attrs, backend} and returns TensorInfo or a list of them
(kernel_registry.ts:55-76).
"""

_KERNELS = {}


class KernelConfig(object):
    __slots__ = ("kernelName", "backendName", "kernelFunc", "setupFunc", "disposeFunc")

    def __init__(self, kernelName, backendName, kernelFunc, setupFunc=None, disposeFunc=None):
        self.kernelName = kernelName
        self.backendName = backendName
        self.kernelFunc = kernelFunc
        self.setupFunc = setupFunc
        self.disposeFunc = disposeFunc


def _key(kernel_name, backend_name):
    return "%s_%s" % (backend_name, kernel_name)


def register_kernel(config):
    """kernel_registry.ts:131-140 (a duplicate registration only warns there)."""
    _KERNELS[_key(config.kernelName, config.backendName)] = config


def get_kernel(kernel_name, backend_name):
    """kernel_registry.ts:88-92."""
    return _KERNELS.get(_key(kernel_name, backend_name))


def get_kernels_for_backend(backend_name):
    """kernel_registry.ts:100-112."""
    return [c for c in _KERNELS.values() if c.backendName == backend_name]


def unregister_kernel(kernel_name, backend_name):
    key = _key(kernel_name, backend_name)
    if key not in _KERNELS:
        raise ValueError("The kernel '%s' for backend '%s' is not registered" %
                         (kernel_name, backend_name))
    del _KERNELS[key]
