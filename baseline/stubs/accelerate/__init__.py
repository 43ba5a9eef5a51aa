"""Stand-in for `accelerate`, which this image lacks.  The reference uses one function of it,
`init_empty_weights`, to build its module tree without memory for the parameters before it assigns the
loaded tensors."""

import contextlib

import torch


@contextlib.contextmanager
def init_empty_weights(include_buffers: bool = False):
    """Parameters registered inside the block are moved to the meta device; buffers (the reference's rotary
    tables) only with ``include_buffers``."""
    register_parameter = torch.nn.Module.register_parameter
    register_buffer = torch.nn.Module.register_buffer

    def parameter_on_meta(module, name, param):
        if param is not None:
            param = torch.nn.Parameter(param.detach().to("meta"), requires_grad=param.requires_grad)
        register_parameter(module, name, param)

    def buffer_on_meta(module, name, tensor, persistent=True):
        if tensor is not None:
            tensor = tensor.to("meta")
        register_buffer(module, name, tensor, persistent=persistent)

    torch.nn.Module.register_parameter = parameter_on_meta
    if include_buffers:
        torch.nn.Module.register_buffer = buffer_on_meta
    try:
        yield
    finally:
        torch.nn.Module.register_parameter = register_parameter
        torch.nn.Module.register_buffer = register_buffer
