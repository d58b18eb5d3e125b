"""A small Engine with the part of tfjs-core/src/engine.ts this backend plugs
into: backend registration by priority, kernel lookup and dispatch, tensor
handles, and the IS_TEST data-id leak check.

In a Node deployment tfjs-core's own Engine plays this role unchanged; this
module exists so the same kernels, registered the same way, can be driven from
Python (tests, benchmark, graph runner).
"""
import numpy as np

from . import kernel_registry
from .backend import TensorInfo


class Tensor(object):
    """Handle over {dataId, shape, dtype} (tfjs-core/src/tensor.ts)."""

    def __init__(self, engine, info):
        self._engine = engine
        self.dataId = info.dataId
        self.shape = list(info.shape)
        self.dtype = info.dtype
        self.isDisposed = False

    @property
    def rank(self):
        return len(self.shape)

    @property
    def size(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    def info(self):
        return TensorInfo(self.dataId, self.shape, self.dtype)

    def dataSync(self):
        """engine.ts:1218-1222 -> backend.readSync."""
        self._check()
        return self._engine.backend.readSync(self.dataId)

    def data(self, into=None):
        """tensor.data(): Promise (tensor.ts:322-336 -> backend.read).  Returns a
        PendingRead; `.wait()` yields the values.  Kernels launched after this call
        run while the copy is outstanding."""
        self._check()
        return self._engine.backend.read(self.dataId, into)

    def arraySync(self):
        return self.dataSync().reshape(self.shape)

    def dispose(self):
        """engine.ts:917-943."""
        if self.isDisposed:
            return
        self.isDisposed = True
        self._engine.dispose_tensor(self)

    def _check(self):
        if self.isDisposed:
            raise RuntimeError("Tensor is disposed.")

    def __repr__(self):
        return "Tensor(shape=%s, dtype=%s)" % (self.shape, self.dtype)


class Engine(object):
    def __init__(self):
        self.registry_factory = {}   # name -> (factory, priority)
        self.registry = {}           # name -> backend instance
        self.backend_name = None
        self.backend = None
        self.num_tensors = 0
        self.is_test = False
        self._profile = None   # list of kernel records while tf.profile is active
        self._prof_stack = []  # records of the kernel funcs being executed
        self._prof_next_slot = 0

    # ---------------------------------------------------------- backends --
    def register_backend(self, name, factory, priority=1):
        """engine.ts:260-272."""
        if name in self.registry_factory:
            return False
        self.registry_factory[name] = (factory, priority)
        return True

    def set_backend(self, name):
        """engine.ts:274-293, 319-369."""
        if name not in self.registry_factory:
            raise ValueError("Backend name '%s' not found in registry" % name)
        if name not in self.registry:
            factory, _ = self.registry_factory[name]
            self.registry[name] = factory()
            for cfg in kernel_registry.get_kernels_for_backend(name):
                if cfg.setupFunc is not None:
                    cfg.setupFunc(self.registry[name])
        self.backend_name = name
        self.backend = self.registry[name]
        return True

    def ready(self):
        """engine.ts:408-422: the highest-priority backend that initialises."""
        if self.backend is not None:
            return self.backend
        errors = []
        for name, _ in sorted(self.registry_factory.items(), key=lambda kv: -kv[1][1]):
            try:
                self.set_backend(name)
                return self.backend
            except Exception as e:  # initialisation failed: try the next one
                errors.append("%s: %s" % (name, e))
        raise RuntimeError("Could not initialize any backends, all backend "
                           "initializations failed. " + "; ".join(errors))

    def remove_backend(self, name):
        """engine.ts:371-392."""
        if name in self.registry:
            self.registry[name].dispose()
            del self.registry[name]
        self.registry_factory.pop(name, None)
        if self.backend_name == name:
            self.backend_name = None
            self.backend = None

    # ----------------------------------------------------------- tensors --
    def make_tensor(self, values, shape=None, dtype=None):
        """engine.ts:803-827 -> backend.write."""
        self.ready()
        arr = np.asarray(values)
        if dtype is None:
            if arr.dtype == np.bool_:
                dtype = "bool"
            elif np.issubdtype(arr.dtype, np.integer):
                dtype = "int32"
            else:
                dtype = "float32"
        if shape is None:
            shape = list(arr.shape)
        data_id = self.backend.write(arr, shape, dtype)
        self.num_tensors += 1
        return Tensor(self, TensorInfo(data_id, shape, dtype))

    def make_tensor_from_info(self, info):
        """engine.ts:848-854."""
        self.num_tensors += 1
        return Tensor(self, info)

    def dispose_tensor(self, t):
        self.num_tensors -= 1
        self.backend.disposeData(t.dataId)

    def memory(self):
        """engine.ts:959-974."""
        info = {"numTensors": self.num_tensors, "numDataBuffers": self.backend.numDataIds()}
        info.update(self.backend.memory())
        return info

    # ----------------------------------------------------------- kernels --
    def run_kernel(self, kernel_name, inputs, attrs=None):
        """engine.ts:539-555, 595-744: look the kernel up for the active backend,
        call kernelFunc({inputs, attrs, backend}), wrap outputs in tensors."""
        self.ready()
        kernel = kernel_registry.get_kernel(kernel_name, self.backend_name)
        if kernel is None:
            raise RuntimeError("Kernel '%s' not registered for backend '%s'" %
                               (kernel_name, self.backend_name))
        infos = {k: (v.info() if isinstance(v, Tensor) else v) for k, v in inputs.items()}
        before = self.backend.numDataIds()
        prof = self._profile
        if prof is not None:
            rec = {"name": kernel_name, "slot": self._take_slots(),
                   "inputShapes": {k: list(v.shape) for k, v in infos.items() if v is not None},
                   "attrs": attrs or {}, "parts": [], "nested": []}
            self._prof_stack.append(rec)
            self.backend.event_record(rec["slot"])
        out = kernel.kernelFunc({"inputs": infos, "attrs": attrs or {}, "backend": self.backend})
        if prof is not None:
            self.backend.event_record(rec["slot"] + 1)
            # what tfjs-core's profiler prints as the kernel's extra information
            # (profiler.ts:74-76): the kernel instantiations this call launched
            rec["extraInfo"] = ", ".join(t for t in rec.pop("_extra", []) +
                                         [self.backend.launch_log_take()] if t)
            self._prof_stack.pop()
            o = out if isinstance(out, (list, tuple)) else [out]
            rec["outputShapes"] = [list(t.shape) for t in o]
            # a kernel whose launch was deferred shows up later, as `parts` of the
            # record in which it was launched
            rec["deferred"] = any(self.backend.pending_of(t.dataId) is not None for t in o)
            prof.append(rec)
        outs = out if isinstance(out, (list, tuple)) else [out]
        if self.is_test:
            # engine.ts:557-588: a kernel may only add one data id per output
            # whose data id is new.
            in_ids = set(id(i.dataId) for i in infos.values() if i is not None)
            new = len(set(id(o.dataId) for o in outs if id(o.dataId) not in in_ids))
            leaked = self.backend.numDataIds() - before - new
            if leaked > 0:
                raise RuntimeError("Backend '%s' has an internal memory leak (%d data ids) "
                                   "after running '%s'" % (self.backend_name, leaked, kernel_name))
        tensors = [self.make_tensor_from_info(o) for o in outs]
        return tensors if isinstance(out, (list, tuple)) else tensors[0]


    def _take_slots(self):
        slot = self._prof_next_slot
        self._prof_next_slot += 2
        return slot

    def deferred_launch(self, descs, launch, fold_into_caller):
        """Called by the backend while profiling when it launches deferred kernels
        (`descs`: their would-be records).  A launch folded into the calling kernel
        (an activation joining its producer) becomes part of the caller's record;
        a launch that merely had to happen first gets a record of its own and its
        time is taken out of the caller's."""
        if fold_into_caller and self._prof_stack:
            self._prof_stack[-1]["parts"] = list(descs)
            self._prof_stack[-1]["folded"] = True
            return launch()
        rec = {"slot": self._take_slots(), "inputShapes": {}, "attrs": {}, "nested": [],
               "deferred": False}
        # launches noted so far belong to the kernel func that is running
        if self._prof_stack:
            self._prof_stack[-1].setdefault("_extra", []).append(self.backend.launch_log_take())
        self.backend.event_record(rec["slot"])
        self._prof_stack.append(rec)      # launches of pending operands nest under this one
        try:
            result = launch()
        finally:
            self._prof_stack.pop()
        self.backend.event_record(rec["slot"] + 1)
        rec["extraInfo"] = ", ".join(t for t in rec.pop("_extra", []) +
                                     [self.backend.launch_log_take()] if t)
        # a launch may narrow `descs` to what it really covered (a chain that ran as its
        # last kernel only), so the record is named afterwards
        rec.update(name="+".join(d["name"] for d in descs), parts=list(descs),
                   outputShapes=descs[-1]["outputShapes"])
        if self._prof_stack:
            self._prof_stack[-1]["nested"].append(rec["slot"])
        self._profile.append(rec)
        return result

    def profile(self, f):
        """tf.profile (engine.ts:976-998): runs f and returns one record per kernel
        with its name, shapes and device time (`kernelTimeMs`, from CUDA events
        recorded on the backend's stream around each kernel func)."""
        self.ready()
        self._profile = []
        self._prof_stack = []
        self._prof_next_slot = 0
        self.backend.profiler = self
        self.backend.launch_log(True)
        try:
            result = f()
        finally:
            records, self._profile = self._profile, None
            self.backend.profiler = None
            self.backend.launch_log(False)
        for rec in records:
            ms = self.backend.event_elapsed(rec["slot"], rec["slot"] + 1)
            for slot in rec["nested"]:
                ms -= self.backend.event_elapsed(slot, slot + 1)
            rec["kernelTimeMs"] = max(ms, 0.0)
            if rec.get("folded"):
                rec["name"] = "+".join([d["name"] for d in rec["parts"]] + [rec["name"]])
        return {"kernels": records, "result": result}


ENGINE = Engine()
