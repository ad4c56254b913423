"""Parallelism strategies built on the put/signal substrate: expert and tensor parallel."""
from .ep import ExpertParallelLayer
from .tp import AllGatherGemm, GemmReduceScatter, LocalTpGroup
