"""One output of the loader: a source field, its decoder and the transforms after it
(reference: ``ffcv/pipeline/pipeline_spec.py:8-50``)."""
from typing import List, Union

import torch as ch

from .operation import Operation


class PipelineSpec:
    def __init__(self, source: Union[str, Operation], decoder: Operation = None,
                 transforms: List[Operation] = None):
        self.source = source
        self.decoder = decoder
        self.transforms = list(transforms) if transforms is not None else []
        self.default_pipeline = decoder is None and not self.transforms and isinstance(source, str)

    def __repr__(self):
        return repr((self.source, self.decoder, self.transforms))

    def accept_decoder(self, Decoder, output_name):
        from ..transforms.module import ModuleWrapper
        from ..transforms.ops import ToTensor
        if not isinstance(self.source, str) and self.decoder is not None:
            raise ValueError("Source can't be a node and also have a decoder")
        if Decoder is not None:
            if self.transforms and isinstance(self.transforms[0], Decoder):
                self.decoder = self.transforms.pop(0)
            elif self.decoder is None:
                try:
                    self.decoder = Decoder()
                except Exception:
                    raise ValueError(f"Impossible to use default decoder for {output_name},"
                                     "make sure you specify one in your pipeline.")
        if self.default_pipeline:
            self.transforms.append(ToTensor())
        for i, op in enumerate(self.transforms):
            if isinstance(op, ch.nn.Module):
                self.transforms[i] = ModuleWrapper(op)
