"""Host-side components for heterogeneous placement: shared-memory request/response channel to an expert server
process, a shared host arena for expert weights, the CPU expert server loop, and the KV quantiser prototype."""
