"""Small shared helpers: seeded fills, scaled closeness, contained child processes (crates/poot-test-util/src/lib.rs:1-9)."""
from .testing import assert_close_scaled, run_contained, seeded_fill
