// C shim around the reference's header-only flag-word helpers
// (src/dynamic_launch_utils.hpp:10-41) so that tests can call the reference's
// own code.  The header is included from the reference tree at build time;
// nothing from it is copied here.
#define __device__
#define __host__
#include REF_FLAG_HEADER

extern "C" {
int ref_set_gemm_flag(int flag, int mode) {
  cumpsgemm::dynamic_launch::utils::set_gemm_flag(flag, mode);
  return flag;
}
int ref_set_scale_A_flag(int flag, int enable) {
  cumpsgemm::dynamic_launch::utils::set_scale_A_flag(flag, enable != 0);
  return flag;
}
int ref_set_scale_B_flag(int flag, int enable) {
  cumpsgemm::dynamic_launch::utils::set_scale_B_flag(flag, enable != 0);
  return flag;
}
int ref_get_gemm_flag(int flag) { return cumpsgemm::dynamic_launch::utils::get_gemm_flag(flag); }
int ref_get_scale_A_flag(int flag) {
  return cumpsgemm::dynamic_launch::utils::get_scale_A_flag(flag) ? 1 : 0;
}
int ref_get_scale_B_flag(int flag) {
  return cumpsgemm::dynamic_launch::utils::get_scale_B_flag(flag) ? 1 : 0;
}
}
