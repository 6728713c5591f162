"""``WebDNN.load`` and ``RunnerImpl`` for the Python host mirror.

``load()`` follows ``src/descriptor_runner/index.ts:42-149``: a cpu context always exists, each
name of ``backendOrder`` is tried in turn, the first that initialises wins, and the runner is built
with ``[succeeded, "cpu"]``.  Only ``"cuda"`` and ``"cpu"`` exist here.

``Runner.run()`` restates ``core/runnerImpl.ts:315-596`` step by step: seed the per-backend tensor
maps with initializers (and the device copies cached from earlier runs), bind inputs positionally,
compute release timing, then for each node find where its inputs live, instantiate the operator,
move inputs according to its backend requirement, run it, file its outputs under their backend and
dispose tensors after their last consumer; finally move outputs to the cpu and dispose the rest.

One deliberate difference: the reference retries a failing node once on the cpu backend
(``runnerImpl.ts:511-520``).  This backend ships no cpu implementation of the arithmetic ops, so a
node that fails on ``cuda`` raises; ``node_backends`` of the last run is exposed so callers can
assert that nothing ran on the host except shape bookkeeping.
"""
from __future__ import annotations

import ctypes
import json
import logging
import os
import time
from typing import Dict, List, Optional, Sequence, Union

import numpy as np

from . import onnx_io, tensor_loader
from .backend import CPUTensor, EightbitCPUTensor, WebDNNCPUContext, WebDNNCudaContext
from .model_transform import find_tensor_release_timing, model_transform
from .onnx_io import FLOAT, INT32, INT64, Model, clip_long
from .tensor_loader import TensorLoader
from .operator_table import instantiate_operator, register_operators, registered_op_types

logger = logging.getLogger("WebDNN.runner")

BACKENDS = ["cpu", "cuda"]
BACKENDS_WITHOUT_CPU = ["cuda"]

_registered_backends = set()


def _register(backend: str) -> None:
    if backend in _registered_backends:
        return
    if backend == "cpu":
        from .operators.host import get_op_entries
    else:
        from .operators.cuda import get_op_entries
    register_operators(get_op_entries())
    _registered_backends.add(backend)


class Runner:
    def __init__(self, backend_order: Sequence[str], backend_contexts: Dict[str, object]):
        self.backend_order = list(backend_order)
        self.backend_contexts = backend_contexts
        self.model: Optional[Model] = None
        self.loaded = False
        self.opset = 0
        self.initializer_tensors: Dict[str, CPUTensor] = {}
        self.copied_initializer_tensors: Dict[str, Dict[str, object]] = {b: {} for b in BACKENDS_WITHOUT_CPU}
        self.tensor_move_options: Dict[str, dict] = {}
        self.force_operator_backend_order: Dict[str, List[str]] = {}
        self.inputs_without_initializer = []
        self.node_backends: List[tuple] = []      # (node name, op type, backend) of the last run
        self.node_performances: List[dict] = []
        # backendOptions.cuda.graphReplay: the second run() with host inputs of a given signature (shapes and
        # dtypes) is recorded as a CUDA graph, and every later run() with that signature replays it
        self.graph_replay = False
        # backendOptions.cuda.graphReplay = "auto" (the default): replay only runs whose inputs all have a leading
        # dimension of at most GRAPH_REPLAY_AUTO_BATCH, where the host's per-node work is as long as the GPU's
        self.graph_replay_auto = False
        self.graph_replays = 0                    # run() calls served by a replay
        self._captured: Dict[tuple, "CapturedRun"] = {}
        self._seen: Dict[tuple, int] = {}
        self._uncapturable = False
    MAX_CAPTURED_SIGNATURES = 4                   # each recorded run keeps its own activation memory
    GRAPH_REPLAY_AUTO_BATCH = 32

    def _replay_wanted(self, inputs) -> bool:
        if self.graph_replay:
            return True
        return self.graph_replay_auto and all(len(t.dims) > 0 and t.dims[0] <= self.GRAPH_REPLAY_AUTO_BATCH
                                              for t in inputs)

    # ---- runnerImpl.ts:88-134
    DEVICE_DECODE_MIN_ELEMENTS = 4096  # 8-bit initializers at least this large are decoded on the device

    def load_model(self, source: Union[str, bytes, Model], onnx_basename: str = "model.onnx") -> None:
        if isinstance(source, Model):
            model = onnx_io.decode_model(onnx_io.encode_model(source))  # private copy
        elif isinstance(source, (bytes, bytearray)):
            model = onnx_io.decode_model(bytes(source))
        else:
            path = os.path.join(source, onnx_basename) if os.path.isdir(source) else source
            model = onnx_io.load_model(path)
        # external initializers (runnerImpl.ts:235-270): "WebDNN2.WeightPaths" names the parts of one
        # WDN2 container beside the model.  Small or uncompressed tensors join the graph's own
        # initializers before the load-time rewrite (which folds BatchNormalization parameters);
        # large 8-bit ones stay as codes and are expanded on the device when first moved there.
        lazy = []
        weight_paths = model.metadata_props.get("WebDNN2.WeightPaths")
        if weight_paths and isinstance(source, str):
            directory = source if os.path.isdir(source) else os.path.dirname(source)
            loader = TensorLoader([os.path.join(directory, bn) for bn in weight_paths.split(":")],
                                  self.backend_contexts["cpu"])
            own = {t.name: i for i, t in enumerate(model.graph.initializer)}
            for rec in loader.records():
                if rec.compression == 1 and "cuda" in self.backend_order and rec.numel >= self.DEVICE_DECODE_MIN_ELEMENTS:
                    lazy.append(rec)
                    continue
                t = onnx_io.make_tensor(rec.name, tensor_loader.decode(rec).reshape(rec.dims))
                if rec.name in own:
                    model.graph.initializer[own[rec.name]] = t
                else:
                    model.graph.initializer.append(t)
        model_transform(model, self.backend_order)
        if not model.opset_import:
            raise ValueError("opsetImport is empty")
        self.opset = int(model.opset_import[0][1])
        self.model = model
        self.initializer_tensors = self._extract_initializer_tensor()
        for rec in lazy:
            codes, scale = tensor_loader.eightbit_codes(rec)
            self.initializer_tensors[rec.name] = EightbitCPUTensor(rec.dims, codes, scale)
        for md_key, md_value in model.metadata_props.items():
            if md_key == "WebDNN2.TensorMoveOptions":
                self.tensor_move_options = json.loads(md_value)
            elif md_key == "WebDNN2.ForceOperatorBackendOrder":
                self.force_operator_backend_order = json.loads(md_value)
        init_names = set(self.initializer_tensors)
        self.inputs_without_initializer = [vi for vi in model.graph.input if vi.name not in init_names]
        self.loaded = True

    # ---- runnerImpl.ts:136-233
    def _extract_initializer_tensor(self) -> Dict[str, CPUTensor]:
        tensors: Dict[str, CPUTensor] = {}
        cpu = self.backend_contexts["cpu"]
        for t in self.model.graph.initializer:
            dims = [clip_long(int(d)) for d in t.dims]
            if t.data_type == FLOAT:
                tensors[t.name] = cpu.empty_tensor(dims, "float32", np.ascontiguousarray(t.array, dtype=np.float32))
            elif t.data_type == INT64:
                arr = np.clip(t.array.astype(np.int64), -(2 ** 31), 2 ** 31 - 1).astype(np.int32)
                tensors[t.name] = cpu.empty_tensor(dims, "int32", arr)
            elif t.data_type == INT32:
                tensors[t.name] = cpu.empty_tensor(dims, "int32", np.ascontiguousarray(t.array, dtype=np.int32))
            else:
                raise ValueError(f"Unsupported initializer dataType {t.data_type}")
        return tensors

    def capture(self, inputs: Sequence[CPUTensor]) -> CapturedRun:
        """Records ``run(inputs)`` on the cuda backend as a CUDA graph.  The run is executed once
        normally first (constants are moved, packed and split then), and the recorded run must stay on
        the device: a node placed on the cpu backend, or an operator that uploads host data while it
        runs (Pad / Tile index tables), ends the capture with an error."""
        ctx = self.backend_contexts.get("cuda")
        if ctx is None:
            raise RuntimeError("capture needs the cuda backend")
        dev_in = []
        for t in inputs:
            if t.backend == "cpu":
                dev_in.append(ctx.move_tensor(t))
            else:   # a device tensor (e.g. a prefetched batch): the recorded run gets its own input buffer
                ctx.wait_upload(t)
                own = ctx.empty_tensor(t.dims, t.data_type)
                ctx._call("wdc_copy", ctypes.c_void_p(own.ptr), ctypes.c_void_p(t.ptr), own.length * 4)
                dev_in.append(own)
        for o in self.run(dev_in, outputs_on_device=True):
            o.dispose()
        if self.nodes_on("cpu"):
            for t in dev_in:
                t.dispose()
            raise RuntimeError(f"capture: nodes on the cpu backend: {self.nodes_on('cpu')}")
        ctx.sync()
        ctx.capture_begin()
        try:
            outs = self.run(dev_in, outputs_on_device=True)
        except Exception:
            try:
                ctx.capture_end()
            except Exception:
                pass
            for t in dev_in:
                t.dispose()
            raise
        graph = ctx.capture_end()
        return CapturedRun(ctx, graph, dev_in, outs)

    def get_input_names(self) -> List[str]:
        return [vi.name for vi in self.inputs_without_initializer]

    def get_output_names(self) -> List[str]:
        return [vi.name for vi in self.model.graph.output]

    # ---- runnerImpl.ts:315-596
    def run(self, inputs: Sequence[CPUTensor], measure_performance: bool = False,
            outputs_on_device: bool = False, wait: bool = True):
        """``inputs`` are CPUTensors as in the reference; a tensor that already lives on a device
        backend is filed under that backend instead (used to time the device path with resident
        inputs).  ``outputs_on_device`` skips the final move to the cpu and returns the device
        tensors, which the caller must dispose.  ``wait=False`` returns a ``PendingRun`` at once: the
        kernels and the device-to-host transfer of the outputs are queued, ``PendingRun.result()`` waits for
        them and returns the CPU tensors, so a caller can queue the next run before it reads this one
        (the reference's run() is a promise the caller awaits: the counterpart of awaiting it later)."""
        if self.model is None or not self.loaded:
            raise RuntimeError("not initialized")
        if not wait:
            return self._run_pending(inputs)
        if (self._replay_wanted(inputs) and not measure_performance and not outputs_on_device
                and len(inputs) == len(self.inputs_without_initializer)
                and all(t.backend == "cpu" or (t.backend == "cuda" and getattr(t, "layout", "nchw") == "nchw")
                        for t in inputs)):
            sig = tuple((tuple(t.dims), t.data_type) for t in inputs)
            cap = self._captured.get(sig)
            if cap is None and not self._uncapturable and self._seen.get(sig, 0) >= 1 \
                    and len(self._captured) < self.MAX_CAPTURED_SIGNATURES:
                try:
                    cap = self._captured[sig] = self.capture(inputs)
                except Exception as e:   # e.g. a node on the cpu backend: keep running node by node
                    logger.warning("graph replay disabled for this runner: %s", e)
                    self._uncapturable = True
            if cap is not None:
                self.graph_replays += 1
                return cap.run(inputs)
            self._seen[sig] = self._seen.get(sig, 0) + 1
        graph = self.model.graph
        tensors_for_backends: Dict[str, Dict[str, object]] = {b: {} for b in BACKENDS}
        for name, tensor in self.initializer_tensors.items():
            tensors_for_backends["cpu"][name] = tensor
        for backend, kv in self.copied_initializer_tensors.items():
            for name, tensor in kv.items():
                tensors_for_backends[backend][name] = tensor

        if len(self.inputs_without_initializer) != len(inputs):
            raise ValueError("length of inputs mismatch")
        borrowed = set()
        for vi, t in zip(self.inputs_without_initializer, inputs):
            tensors_for_backends[t.backend][vi.name] = t
            if t.backend != "cpu":
                borrowed.add(vi.name)  # caller-owned device tensor: never disposed here
                wait = getattr(self.backend_contexts.get(t.backend), "wait_upload", None)
                if wait is not None:
                    wait(t)  # a prefetched input: order the first kernel after its transfer

        release_timing = find_tensor_release_timing(self.model, set(self.initializer_tensors))
        self.node_backends = []
        self.node_performances = []

        for node in graph.node:
            t0 = time.perf_counter()
            op_type = node.op_type
            order = self.force_operator_backend_order.get(node.name) or self.backend_order
            current: List[List[str]] = []
            for input_name in node.input:
                bs = [b for b in order if input_name in tensors_for_backends[b]]
                if not bs:
                    bs = [b for b in BACKENDS if input_name in tensors_for_backends[b]]
                current.append(bs)
            operator = instantiate_operator(op_type, self.opset, order, current)
            if operator is None:
                raise RuntimeError(f"Operator implementation for {op_type}, opset={self.opset} does not exist.")
            operator.initialize(node.attribute)
            requirement = operator.get_tensor_backend_requirement(len(node.input), len(node.output))
            operator_inputs = []
            for j, input_name in enumerate(node.input):
                req = requirement[j]
                if not req:
                    if not current[j]:
                        raise RuntimeError(f"Input {input_name} not found")
                    operator_inputs.append(tensors_for_backends[current[j][0]][input_name])
                    continue
                t = tensors_for_backends[req].get(input_name)
                if t is not None:
                    operator_inputs.append(t)
                    continue
                for other in self.backend_order:
                    other_t = tensors_for_backends[other].get(input_name)
                    if other_t is not None:
                        moved = self.backend_contexts[req].move_tensor(
                            other_t, self.tensor_move_options.get(input_name, {}))
                        tensors_for_backends[req][input_name] = moved
                        operator_inputs.append(moved)
                        break
                else:
                    raise RuntimeError(f"Input {input_name} not found")
            context = self.backend_contexts[operator.backend]
            logger.debug("Running %s(%s) on %s", node.name, op_type, operator.backend)
            ranged = getattr(context, "profile", False)
            if ranged:
                context.range_push(f"{node.name}({op_type})")
            try:
                outputs = operator.run(context, operator_inputs, len(node.output))
            finally:
                if ranged:
                    context.range_pop()
            for j, output_name in enumerate(node.output):
                tensors_for_backends[outputs[j].backend][output_name] = outputs[j]
            self.node_backends.append((node.name, op_type, operator.backend))

            for name in release_timing.get(node.name, []):
                for backend in BACKENDS:
                    t = tensors_for_backends[backend].pop(name, None)
                    if t is not None:
                        t.dispose()
            if measure_performance:
                sync = getattr(context, "sync", None)
                if sync is not None:
                    sync()  # device backends only enqueue: wait, so that elapsed is this node's time
                self.node_performances.append(dict(
                    opType=op_type, name=node.name, backend=operator.backend,
                    inputDims=[t.dims for t in operator_inputs], outputDims=[t.dims for t in outputs],
                    elapsed=(time.perf_counter() - t0) * 1e3))

        results: List[CPUTensor] = []
        kept = set()
        for vi in graph.output:
            out = tensors_for_backends["cpu"].get(vi.name)
            if out is None and outputs_on_device:
                for other in self.backend_order:
                    out = tensors_for_backends[other].get(vi.name)
                    if out is not None:
                        kept.add(vi.name)
                        break
            if out is None:
                for other in self.backend_order:
                    other_t = tensors_for_backends[other].get(vi.name)
                    if other_t is not None:
                        out = self.backend_contexts["cpu"].move_tensor(other_t, {})
                        tensors_for_backends["cpu"][vi.name] = out
                        break
            if out is None:
                raise RuntimeError(f"Output {vi.name} not found")
            results.append(out)

        for backend in BACKENDS_WITHOUT_CPU:
            for name, t in tensors_for_backends[backend].items():
                if name in self.initializer_tensors:
                    self.copied_initializer_tensors[backend][name] = t
                elif name not in borrowed and name not in kept:
                    t.dispose()
        return results

    def _run_pending(self, inputs) -> "PendingRun":
        ctx = self.backend_contexts.get("cuda")
        if ctx is None:
            return PendingRun(None, [], [], ready=self.run(inputs))
        cap = None
        replay = self._replay_wanted(inputs)
        if replay and len(inputs) == len(self.inputs_without_initializer):
            cap = self._captured.get(tuple((tuple(t.dims), t.data_type) for t in inputs))
        if cap is not None:
            self.graph_replays += 1
            cap.load_inputs(inputs)
            cap.launch()
            # the recorded output buffers are overwritten by the next replay: the transfer reads a private copy
            outs = []
            for o in cap.outputs:
                c = ctx.empty_tensor(o.dims, o.data_type)
                src = ctx.canonical(o)
                ctx._call("wdc_copy", ctypes.c_void_p(c.ptr), ctypes.c_void_p(src.ptr), o.length * 4)
                if src is not o:
                    src.dispose()
                outs.append(c)
        else:
            if replay and not self._uncapturable:   # the ordinary path records the graph on its second use of a signature
                first = self.run(inputs)
                return PendingRun(None, [], [], ready=first)
            outs = self.run(inputs, outputs_on_device=True)
        downloads = [ctx.download_async(o) if getattr(o, "backend", "cpu") == "cuda" else None for o in outs]
        return PendingRun(ctx, outs, downloads)

    def nodes_on(self, backend: str) -> List[tuple]:
        return [n for n in self.node_backends if n[2] == backend]

    def dispose(self) -> None:
        for cap in self._captured.values():
            cap.dispose()
        self._captured.clear()
        for kv in self.copied_initializer_tensors.values():
            for t in kv.values():
                t.dispose()
            kv.clear()


class PendingRun:
    """Outputs of a ``Runner.run(..., wait=False)`` whose kernels and device-to-host transfers are queued."""

    def __init__(self, context, device_outputs, downloads, ready=None):
        self.context, self.device_outputs, self.downloads, self.ready = context, device_outputs, downloads, ready

    def result(self) -> List[CPUTensor]:
        if self.ready is not None:
            return self.ready
        outs = []
        for t, d in zip(self.device_outputs, self.downloads):
            if d is None:
                outs.append(t)            # an output that was produced on the cpu backend
                continue
            outs.append(self.context.cpu_context.empty_tensor(t.dims, t.data_type, d.result()))
            t.dispose()
        self.ready = outs
        self.device_outputs, self.downloads = [], []
        return outs


class CapturedRun:
    """One ``Runner.run`` recorded as a CUDA graph (``Runner.capture``): every later ``run`` copies the
    inputs into the recorded input buffers, replays all launches with one call and reads the outputs
    back.  Valid for inputs of the shapes and dtypes given at capture time; the recorded buffers belong
    to this object until ``dispose``."""

    def __init__(self, context: WebDNNCudaContext, graph: int, inputs: List, outputs: List):
        self.context, self.graph, self.inputs, self.outputs = context, graph, inputs, outputs

    def launch(self) -> None:
        """Replay on the inputs currently in the recorded input buffers; results stay on the device."""
        self.context.graph_launch(self.graph)

    def run(self, inputs: Sequence[CPUTensor]) -> List[CPUTensor]:
        if len(inputs) != len(self.inputs):
            raise ValueError("length of inputs mismatch")
        self.load_inputs(inputs)
        self.launch()
        return [self.context.cpu_context.empty_tensor(o.dims, o.data_type, o.get_data()) for o in self.outputs]

    def load_inputs(self, inputs: Sequence[CPUTensor]) -> None:
        if len(inputs) != len(self.inputs):
            raise ValueError("length of inputs mismatch")
        for dst, src in zip(self.inputs, inputs):
            if list(src.dims) != list(dst.dims) or src.data_type != dst.data_type:
                raise ValueError("CapturedRun.run: input shape or dtype differs from the captured one")
            if src.backend == "cpu":
                dst.set_data(src.get_data())
            else:
                # a batch already on the device (moved there by prefetch_tensor while the previous run computed):
                # order after its transfer, then a device-to-device copy into the recorded input buffer
                self.context.wait_upload(src)
                self.context._call("wdc_copy", ctypes.c_void_p(dst.ptr), ctypes.c_void_p(src.ptr), dst.length * 4)

    def dispose(self) -> None:
        if self.graph is None:
            return
        self.context.sync()
        for t in self.outputs:
            t.dispose()
        self.context.graph_destroy(self.graph)
        self.graph = None
        for t in self.inputs:
            t.dispose()


def load(source: Union[str, bytes, Model], backend_order: Optional[Sequence[str]] = None,
         backend_options: Optional[dict] = None, onnx_basename: str = "model.onnx") -> Runner:
    """``WebDNN.load(directory, {backendOrder, backendOptions})`` (index.ts:42-149)."""
    backend_order = list(backend_order) if backend_order is not None else ["cuda", "cpu"]
    backend_options = backend_options or {}
    cpu_context = WebDNNCPUContext()
    _register("cpu")
    contexts: Dict[str, object] = {"cpu": cpu_context}
    succeeded = None
    errors = []
    for name in backend_order:
        if name == "cpu":
            succeeded = "cpu"
            break
        if name != "cuda":
            errors.append(f"unknown backend {name}")
            continue
        try:
            opts = backend_options.get("cuda", {})
            ctx = opts.get("context")
            if ctx is None:
                ctx = WebDNNCudaContext(cpu_context, device=opts.get("device", 0),
                                        arena_bytes=opts.get("arenaBytes", 0))
                ctx.initialize()
            if "precision" in opts:
                ctx.set_precision(opts["precision"])
            if "profile" in opts:
                ctx.profile = bool(opts["profile"])
                ctx.set_option("nvtx", int(ctx.profile))
            contexts["cuda"] = ctx
            _register("cuda")
            succeeded = "cuda"
            break
        except Exception as e:  # index.ts:68-79: try the next backend
            errors.append(f"{name}: {e}")
            logger.warning("backend %s failed to initialise: %s", name, e)
    if succeeded is None:
        raise RuntimeError("No backend available: " + "; ".join(errors))
    order = [succeeded] if succeeded == "cpu" else [succeeded, "cpu"]
    runner = Runner(order, contexts)
    gr = backend_options.get("cuda", {}).get("graphReplay", "auto")
    runner.graph_replay = succeeded == "cuda" and gr is True
    runner.graph_replay_auto = succeeded == "cuda" and gr == "auto"
    runner.load_model(source, onnx_basename)
    return runner
