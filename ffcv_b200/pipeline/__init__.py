from .allocation_query import AllocationQuery
from .compiler import Compiler
from .operation import Operation
from .pipeline_spec import PipelineSpec
from .state import State

__all__ = ['AllocationQuery', 'Compiler', 'Operation', 'PipelineSpec', 'State']
