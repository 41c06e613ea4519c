"""Graph namespace: signature-keyed CUDA-graph caches, the manual capture helper, the install-completeness guard and
(imported on demand: ``graph.dynamo_backend``, ``graph.dynamo_partitioner``) the TorchDynamo front-end."""
from ._runtime import (GraphCache, GraphHandle, GraphSignature, backend_loaded, configure_backend,  # noqa: F401
                       get_default_graph_cache, install_torch_namespace, reset_graph_cache)

from .admission import EntryRegistry, GraphPlan, SignaturePlanner  # noqa: E402,F401
from .manual_capture import GraphCapture, capture  # noqa: E402,F401
from .lazy_init_guard import (DynamoUnsafeLazyStateError, UninitializedLazyStateError, freeze_for_dynamo,  # noqa: E402,F401
                              mark_install_checked, verify_lazy_init)

GraphSignature.__module__ = "rpu_backend.graph"
GraphCache.__module__ = "rpu_backend.graph"

__all__ = ["GraphCache", "GraphSignature", "GraphHandle", "configure_backend", "get_default_graph_cache",
           "reset_graph_cache", "SignaturePlanner", "GraphPlan", "EntryRegistry", "GraphCapture", "capture",
           "verify_lazy_init", "freeze_for_dynamo", "mark_install_checked", "UninitializedLazyStateError",
           "DynamoUnsafeLazyStateError"]
