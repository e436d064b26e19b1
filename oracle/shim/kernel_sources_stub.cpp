// The reference embeds its OpenCL program text in a generated table.  The CPU
// context never compiles a program, so the checker build links an empty table.
#include <map>
#include <string>
namespace dlprim { namespace gpu {
std::map<std::string,std::string> kernel_sources;
}}
