#ifndef SXB_LAMMPS_SHIM_ERROR_H
#define SXB_LAMMPS_SHIM_ERROR_H
#include <string>
namespace LAMMPS_NS {
class Error {
 public:
  template <typename... Args> [[noreturn]] void all(const std::string &, int, const std::string &, Args &&...);
  template <typename... Args> [[noreturn]] void one(const std::string &, int, const std::string &, Args &&...);
};
}
#endif
