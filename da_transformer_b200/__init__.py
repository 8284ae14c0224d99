"""B200-native (sm_100a) replacement of DA-Transformer's ``fs_plugins/custom_ops``.

Re-exports the names of ``fs_plugins/custom_ops/__init__.py`` so that
``from da_transformer_b200 import dag_loss, dag_best_alignment,
dag_logsoftmax_gather_inplace`` is a drop-in for the reference import.
"""
from .dag_loss import (  # noqa: F401
    DagBestAlignmentFunc,
    DagLogsoftmaxGatherFunc,
    DagLossFunc,
    dag_best_alignment,
    dag_logsoftmax_gather_inplace,
    dag_loss,
    get_dag_kernel,
    last_status,
    logsoftmax_gather,
)

from .criterion_glue import dag_loss_mean, dag_match, glat_alignment  # noqa: F401
from .graph_ops import dag_links_from_heads, dag_node_passing_prob, dag_viterbi_decode  # noqa: F401
from .torch_twins import (  # noqa: F401
    torch_dag_best_alignment,
    torch_dag_logsoftmax_gather_inplace,
    torch_dag_loss,
)

__version__ = "0.1.0"
