//! `backend` as it would sit in sage's `src/` (see backend.rs).
pub mod backend;
