"""Parts a model is put together from, and their registries."""

from . import attention, ends, ffn, layer, norm, position  # noqa: F401  (registers the built-in kinds)
from .base import (BuildContext, ParamDecl, Part, Workspace, build_embedding, build_ffn, build_head, build_layer,
                   build_mixer, build_norm, build_position, register_embedding, register_ffn, register_head,
                   register_layer, register_mixer, register_norm, register_position, unregister)

__all__ = ["BuildContext", "ParamDecl", "Part", "Workspace", "build_embedding", "build_ffn", "build_head", "build_layer",
           "build_mixer", "build_norm", "build_position", "register_embedding", "register_ffn", "register_head",
           "register_layer", "register_mixer", "register_norm", "register_position", "unregister"]
