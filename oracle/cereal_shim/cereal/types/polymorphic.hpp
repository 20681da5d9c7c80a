// Stand-in for cereal's polymorphic-registration header.  The registration
// macros expand to nothing: the oracle wrapper never serializes a graph.
// Test infrastructure only.
#pragma once
#define CEREAL_REGISTER_TYPE(T)
#define CEREAL_REGISTER_TYPE_WITH_NAME(T, N)
#define CEREAL_REGISTER_POLYMORPHIC_RELATION(B, D)
