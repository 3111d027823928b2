"""Drop-in name of the PyTorch plugin: ``import flagcx`` registers the
``"flagcx"`` process-group backend, as the reference plugin does
(plugin/torch/flagcx/__init__.py, entry point ``torch.backends: flagcx``).

    import flagcx
    torch.distributed.init_process_group("cpu:gloo,cuda:flagcx", ...)
"""
import flagcx_b200
from flagcx_b200 import register_backend

register_backend("flagcx")


def init():
    """Entry point used by ``torch.backends`` plug-in discovery."""
    register_backend("flagcx")


__all__ = ["init", "register_backend"]
