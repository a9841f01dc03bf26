"""User-facing model object of the ``cuda`` target.

Same surface as the reference's ``AIEModel`` (``src/aie4ml/model.py:29-162``):
``run_pipeline`` / ``write`` / ``build`` / ``compile`` / ``predict(X, simulator, quantize_in,
dequantize_out)``, with ``simulator='cuda'`` as the only executor.  Where the reference writes a
Vitis project and shells out to ``make x86sim`` with text-file I/O
(``src/aie4ml/simulation.py:199-245,337-341``), this object packs constants, allocates HBM, and
launches kernels in-process: quantise -> H2D -> launches -> D2H -> dequantise.
"""

from __future__ import annotations

import json
import logging
from pathlib import Path
from typing import Any, Dict, Optional, Union

import numpy as np

from .ir import BackendContext
from .op_impls.precision import resolve_exact_storage_dtype
from .passes import DEFAULT_PIPELINE, run_aie_passes
from .qtypes import FLOAT_FORMATS
from .quant_utils import (apply_rounding, dequantize, dtype_for_precision, from_storage_float, handle_overflow,
                          to_storage_float)

log = logging.getLogger(__name__)


class CudaModel:
    def __init__(self, ctx: BackendContext, source_model: Optional[Any] = None):
        self._ctx = ctx
        self.source_model = source_model
        self._lowered = False
        self.plan = None
        self._pipeline = None

    # -- reference-compatible surface -------------------------------------------------------------
    @classmethod
    def from_context(cls, ctx: BackendContext, source_model: Optional[Any] = None) -> 'CudaModel':
        return cls(ctx, source_model=source_model)

    @property
    def context(self) -> BackendContext:
        return self._ctx

    def run_pipeline(self) -> 'CudaModel':
        if not self._lowered:
            run_aie_passes(self._ctx, [cls() for cls in DEFAULT_PIPELINE])
            self._lowered = True
        return self

    def write(self) -> 'CudaModel':
        """Lower the graph; when an output directory is configured, also dump the lowered plan
        (``cuda_pipeline.json`` + ``params.npz``), the analogue of ``aie_pipeline.json``."""
        self.run_pipeline()
        out_dir = self._ctx.output_dir
        if out_dir:
            self.dump(out_dir)
        return self

    def build(self, make_target: str = 'all', env=None, log_to_stdout: bool = True) -> int:
        """Pack constants, allocate device memory and build the launch list.  Returns 0."""
        self.run_pipeline()
        if self.plan is None:
            from .runtime import Plan

            fusion = dict(self._ctx.aie_config.get('FusionPolicy', {}) or {})
            self.plan = Plan(self._ctx, fuse_rowop_add=bool(fusion.get('rowop_add', True)),
                             fuse_attention=bool(fusion.get('attention', True)),
                             merge_attention_heads=bool(fusion.get('attention_heads', True)),
                             merge_parallel_dense=bool(fusion.get('parallel_dense', True)),
                             fuse_dense_chain=bool(fusion.get('dense_chain', True)),
                             fuse_dense_ln=bool(fusion.get('dense_ln', True)),
                             dense_algo=int(self._ctx.aie_config.get('DenseAlgo', 0)))
        return 0

    def compile(self) -> int:
        return self.build()

    def predict(self, X, simulator: str = 'cuda', *, quantize_in: bool = True, dequantize_out: bool = True):
        if simulator.lower() != 'cuda':
            raise ValueError(f'Unknown simulator "{simulator}". Expected: cuda.')
        import torch

        self.build()
        plan = self.plan
        graph = self._ctx.ir.logical
        iterations = int(self._ctx.aie_config.get('Iterations', 1))
        prepared = self.prepare_inputs(X, iterations=iterations, quantize=quantize_in)
        outs: Dict[str, list] = {name: [] for name in graph.output_tensor_names}
        if iterations > 1 and all(int(graph.tensors[n].shape[0]) == int(graph.tensors[graph.input_tensor_names[0]].shape[0])
                                  for n in list(graph.input_tensor_names) + list(graph.output_tensor_names)):
            # iterations are chunks of one long batch: copy-in, launches and copy-out overlap across them
            pipe = self.pipeline()
            host_in = {n: _host_tensor(a.reshape(-1, *a.shape[2:]), plan.tensor_of(n).dtype).pin_memory()
                       for n, a in prepared.items()}
            host_out = {}
            for n in outs:
                t = plan.tensor_of(n)
                host_out[n] = torch.empty((iterations * t.shape[0], *t.shape[1:]), dtype=t.dtype).pin_memory()
            pipe.run_and_wait(host_in, host_out)
            for n in outs:
                arr = _host_array(host_out[n])
                outs[n] = list(arr.reshape(iterations, -1, *arr.shape[1:]))
        else:
            for it in range(iterations):
                for name, arr in prepared.items():
                    dst = plan.tensor_of(name)
                    dst.copy_(_host_tensor(arr[it], dst.dtype).to(plan.device, non_blocking=False))
                plan.run()
                plan.check_status()
                for name in outs:
                    outs[name].append(_host_array(plan.tensor_of(name).cpu()))
        result: Dict[str, np.ndarray] = {}
        for name, chunks in outs.items():
            arr = np.stack(chunks, axis=0)
            if dequantize_out and self.tensor_dtype(name).format not in FLOAT_FORMATS:
                arr = dequantize(arr, self.tensor_dtype(name).frac)
            result[name] = arr.reshape(arr.shape[0] * arr.shape[1], *arr.shape[2:]) if arr.ndim >= 2 else arr
        if len(result) == 1:
            return next(iter(result.values()))
        return result

    def pipeline(self, depth: int = 3):
        """The streaming executor for host batches longer than the model's own batch: ``depth`` buffer
        sets, copy-in / launches / copy-out on three streams (see ``streaming.HostPipeline``)."""
        from .streaming import HostPipeline

        self.build()
        if self._pipeline is None or len(self._pipeline.plans) != depth:
            self._pipeline = HostPipeline(self._ctx, depth, first_plan=self.plan)
        return self._pipeline

    # -- helpers ----------------------------------------------------------------------------------
    def tensor_dtype(self, name: str):
        t = self._ctx.ir.logical.tensors[name]
        return resolve_exact_storage_dtype(t.precision, namespace='tensor', layer_name=name)

    def prepare_inputs(self, X, iterations: int = 1, quantize: bool = True) -> Dict[str, np.ndarray]:
        """Shape checking, ``Iterations`` replication and float -> code quantisation of graph inputs
        (reference ``simulation.py:157-196,260-269``)."""
        graph = self._ctx.ir.logical
        names = list(graph.input_tensor_names)
        if len(names) == 1 and not isinstance(X, dict):
            X = {names[0]: X}
        prepared: Dict[str, np.ndarray] = {}
        for name in names:
            expected = tuple(int(s) for s in graph.tensors[name].shape)
            arr = np.asarray(X[name])
            if tuple(arr.shape) == expected:
                arr = np.repeat(arr[np.newaxis, ...], iterations, axis=0)
            elif arr.ndim == len(expected) + 1 and tuple(arr.shape[1:]) == expected and arr.shape[0] == iterations:
                pass
            elif arr.ndim == len(expected) + 1 and tuple(arr.shape[1:]) == expected and arr.shape[0] == 1:
                arr = np.repeat(arr, iterations, axis=0)
            else:
                raise ValueError(f'{name}: expected shape {expected}, (1, *{expected}) or ({iterations}, *{expected}); '
                                 f'got {tuple(arr.shape)}')
            dt = self.tensor_dtype(name)
            if dt.format in FLOAT_FORMATS:
                prepared[name] = to_storage_float(arr, dt.format)[0]   # float-simulation path: a cast, no codes
                continue
            np_dt = dtype_for_precision(dt.width, dt.signed)
            if np.issubdtype(arr.dtype, np.integer):
                prepared[name] = arr.astype(np_dt, copy=False)
            elif quantize:
                scaled = arr.astype(np.float64) * float(1 << max(0, int(dt.frac)))
                codes = apply_rounding(scaled, dt.rounding).astype(np.int64)
                prepared[name] = handle_overflow(codes, dt.width, dt.signed, dt.saturation).astype(np_dt)
            else:
                raise ValueError(f'{name}: quantize=False requires integer inputs')
        return prepared

    def export_plan(self) -> Dict[str, Any]:
        """The lowered plan as plain data (op list with resolved numerics + integer constants)."""
        self.run_pipeline()
        if self.plan is not None:
            return self.plan.export()
        from .runtime import Plan

        return Plan.export(_ExportShim(self._ctx))  # no device needed for an export

    def dump(self, out_dir: Union[str, Path]) -> Path:
        out = Path(out_dir)
        out.mkdir(parents=True, exist_ok=True)
        plan = self.export_plan()
        params = plan.pop('params')
        np.savez(out / 'params.npz', **{k.replace('/', '__'): v for k, v in params.items()})
        (out / 'cuda_pipeline.json').write_text(json.dumps(plan, indent=1, default=str))
        return out / 'cuda_pipeline.json'


def _host_tensor(arr: np.ndarray, dtype=None):
    """NumPy storage array -> torch CPU tensor of the plan tensor's ``dtype`` (bfloat16 arrives as its 16 bits, fp8
    as its 8 bits)."""
    import torch

    arr = np.ascontiguousarray(arr)
    if arr.dtype == np.uint16:
        return torch.from_numpy(arr.view(np.int16)).view(torch.bfloat16)
    if dtype == torch.float8_e4m3fn:
        return torch.from_numpy(arr).view(torch.float8_e4m3fn)
    return torch.from_numpy(arr)


def _host_array(t) -> np.ndarray:
    """torch CPU tensor -> int64 codes, or float32 values for the float-simulation path."""
    import torch

    if t.dtype in (torch.bfloat16, torch.float32, torch.float8_e4m3fn):
        return t.float().numpy()
    return t.numpy().astype(np.int64)


class _ExportShim:
    """Just enough of a Plan for ``Plan.export`` when no device plan has been built."""

    def __init__(self, ctx: BackendContext):
        self.ctx = ctx
        self.graph = ctx.ir.logical
        self.fused: list = []
        self.fmt = {}
        for name, t in self.graph.tensors.items():
            if not t.is_parameter:
                self.fmt[name] = resolve_exact_storage_dtype(t.precision, namespace='tensor', layer_name=name).format


def from_graph(graph_or_builder, config: Optional[Dict[str, Any]] = None) -> CudaModel:
    """Front door for a programmatic ``GraphBuilder``, a graph dict, or a JSON path."""
    from .frontends.graph import GraphBuilder, load_graph_json, lower_graph_dict

    if isinstance(graph_or_builder, GraphBuilder):
        ctx = graph_or_builder.finalize()
    elif isinstance(graph_or_builder, dict):
        ctx = lower_graph_dict(graph_or_builder, config)
    else:
        ctx = load_graph_json(str(graph_or_builder), config)
    return CudaModel.from_context(ctx)
