// Stand-in for a header of the cereal serialization library, which the
// reference pins as a third-party dependency but which is not needed to run
// its MoE arithmetic.  Serialization members in the reference are templates
// that are never instantiated by the oracle wrapper, so an empty header is
// enough to compile against.  Test infrastructure only.
#pragma once
