from unirl_b200.distributed.tensor.batch import (  # noqa: F401
    Batch,
    FieldKind,
    concat_field,
    field,
    max_field,
    mean_field,
    min_field,
    packed_field,
    shared_field,
    sum_field,
)
