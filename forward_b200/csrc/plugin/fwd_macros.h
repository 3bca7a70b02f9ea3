// Namespace macros with the names Forward's sources use (source/common/common_macros.h), so
// the plugin and creator files in this directory drop into Forward's tree unchanged.
#pragma once

#ifndef FWD_NAMESPACE_BEGIN
#define FWD_NAMESPACE_BEGIN namespace fwd {
#define FWD_NAMESPACE_END }
#define FWD_TRT_NAMESPACE_BEGIN namespace fwd { namespace trt_ {
#define FWD_TRT_NAMESPACE_END } }
#define FWD_TORCH_NAMESPACE_BEGIN namespace fwd { namespace torch_ {
#define FWD_TORCH_NAMESPACE_END } }
#endif
