from tinyserve_llm_b200.parts.base import (
    FeedForward,
    KVNeed,
    Mixer,
    Norm,
    Part,
    PositionEncoding,
    Runtime,
    TensorDecl,
    arrangement_class,
    part_class,
    register_arrangement,
    register_part,
)

__all__ = ["FeedForward", "KVNeed", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime", "TensorDecl",
           "arrangement_class", "part_class", "register_arrangement", "register_part"]
