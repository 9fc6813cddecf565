from mlx_lattice_b200.core.relations.specs import KernelSpec
from mlx_lattice_b200.core.relations.views import (
    KernelRelation,
    RelationCSRView,
    RelationEdges,
    RelationImplicitGemmView,
    RelationKind,
    RelationSortedImplicitGemmView,
    SparseRelationContract,
)

__all__ = [
    'KernelRelation',
    'KernelSpec',
    'RelationCSRView',
    'RelationEdges',
    'RelationImplicitGemmView',
    'RelationKind',
    'RelationSortedImplicitGemmView',
    'SparseRelationContract',
]
