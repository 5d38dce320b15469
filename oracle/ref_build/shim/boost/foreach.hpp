// Test infrastructure only: forwards to the standard-library stand-ins.
#include <boost/_shim.hpp>
