"""aie4ml_b200: a B200-native ``cuda`` execution target for aie4ml's lowered, quantized operator graph.

Front doors: :func:`from_graph` (programmatic builder / dict / JSON) and :func:`from_onnx` (when the
``onnx`` package is importable).  Both return a :class:`CudaModel` with the reference's
``write / compile / predict`` surface; execution goes through hand-written sm_100a kernels behind the
C ABI in ``include/aie4ml_b200.h``.
"""

from .frontends.graph import GraphBuilder, intent, lower_graph_dict
from .model import CudaModel, from_graph
from .qtypes import AIEDataType, QuantIntent, RoundingMode, SaturationMode

__version__ = '0.1.0'


def from_onnx(model_or_path, config, *, output_dir=None, project_name=None, **kwargs):
    """ONNX Q/DQ front door (same signature as the reference's ``from_onnx``,
    ``src/aie4ml/frontends/onnx/importer.py:113-130``)."""
    from .frontends.onnx_import import from_onnx as _from_onnx

    return _from_onnx(model_or_path, config, output_dir=output_dir, project_name=project_name, **kwargs)


__all__ = ['AIEDataType', 'CudaModel', 'GraphBuilder', 'QuantIntent', 'RoundingMode', 'SaturationMode', 'from_graph',
           'from_onnx', 'intent', 'lower_graph_dict']
