// Type-only stand-in for <jni.h>, just enough for the reference's native sources to
// compile without a JDK.  Test infrastructure: used only by oracle/build_ref.py when it
// compiles the reference tree into oracle/_ref/.  None of these methods is ever called
// (the wrappers in ref_wrap_*.cu call the reference's C++ dispatchers directly), so they
// are empty.
#pragma once
#include <cstdint>
typedef int32_t jint;
typedef int64_t jlong;
typedef uint8_t jboolean;
typedef int8_t jbyte;
typedef uint16_t jchar;
typedef int16_t jshort;
typedef float jfloat;
typedef double jdouble;
struct _jobject {};
typedef _jobject* jobject;
typedef jobject jclass;
typedef jobject jthrowable;
typedef jobject jstring;
typedef jobject jarray;
typedef jarray jlongArray;
typedef jarray jintArray;
typedef jarray jfloatArray;
typedef jarray jbyteArray;
struct _jmethodID;
typedef _jmethodID* jmethodID;
#define JNIEXPORT
#define JNICALL
#define JNI_TRUE 1
#define JNI_FALSE 0
struct JNIEnv_ {
  jclass FindClass(const char*) { return nullptr; }
  jmethodID GetMethodID(jclass, const char*, const char*) { return nullptr; }
  template <class... T> jobject NewObject(jclass, jmethodID, T...) { return nullptr; }
  jint Throw(jthrowable) { return 0; }
  jstring NewStringUTF(const char*) { return nullptr; }
  void GetLongArrayRegion(jlongArray, jint, jint, jlong*) {}
  void GetIntArrayRegion(jintArray, jint, jint, jint*) {}
  void GetFloatArrayRegion(jfloatArray, jint, jint, jfloat*) {}
  void SetFloatArrayRegion(jfloatArray, jint, jint, const jfloat*) {}
};
typedef JNIEnv_ JNIEnv;
