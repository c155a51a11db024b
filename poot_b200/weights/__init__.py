"""Typed weight vocabulary: roles, ids and the map from ids to stored tensors
(crates/poot-weights/src/role.rs:11-85,178-282, src/map.rs:1-3)."""
from .roles import WeightId, WeightMap, WeightRole, rank_view
